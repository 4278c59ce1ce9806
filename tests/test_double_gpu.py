"""The operators on torch.float64 tensors, as the reference dispatches them
(hingetree.cpp:666-689): checked through the `hingetree_cpp` operators against golden vectors produced by the
unmodified reference in double precision (tests/golden/forest64.npz, written by tests/golden/make_golden.py) and,
where the reference build is at hand (oracle/_ref), against that build itself on larger seeded inputs.

Bars: forward, leaf map, margin map, reachability and the fixed-order backward bit for bit; the default backward
(atomic scatters) within 1e-13 of the summed term magnitudes.
"""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu

DOUBLE = np.load(os.path.join(GOLDEN, "forest64.npz"))


@pytest.fixture(scope="module")
def ext():
    from hingetreefortorch_b200._ext import hingetree_cpp
    return hingetree_cpp


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def check(ext, kind, c):
    x, thr, ord_, w, g = [dev(c[k]) for k in ("x", "thr", "ord", "w", "g")]
    assert x.dtype == torch.float64
    out = getattr(ext, kind + "_forward")(x, thr, ord_, w)
    assert out.dtype == torch.float64 and np.array_equal(out.cpu().numpy(), c["out"], equal_nan=True)
    assert np.array_equal(getattr(ext, kind + "_leafmap")(x, thr, ord_, w).cpu().numpy(), c["leaf"])
    margin, mord = getattr(ext, kind + "_marginmap")(x, thr, ord_, w)
    assert np.array_equal(margin.cpu().numpy(), c["margin"], equal_nan=True) and np.array_equal(mord.cpu().numpy(), c["margin_ord"])
    assert np.array_equal(getattr(ext, kind + "_reachability")(x, thr, ord_, w).cpu().numpy(), c["reach"])
    fixed = getattr(ext, kind + "_backward_deterministic")(x, True, thr, True, ord_, False, w, True, g)
    assert fixed[2] is None
    for got, name in zip((fixed[0], fixed[1], fixed[3]), ("gx", "gthr", "gw")):
        assert np.array_equal(got.cpu().numpy(), c[name], equal_nan=True), name
    # scale of the default mode's tolerance: summed |terms| (taken in single precision: a scale, not a value)
    f32 = [np.asarray(c[k], dtype=np.float32) for k in ("x", "thr")] + [c["ord"]] + [np.asarray(c[k], dtype=np.float32) for k in ("w", "g")]
    mags = ho.backward_magnitudes(kind, *f32)
    free = getattr(ext, kind + "_backward")(x, True, thr, True, ord_, False, w, True, g)
    for got, name, mag in zip((free[0], free[1], free[3]), ("gx", "gthr", "gw"), mags):
        ref = c[name]
        if np.isfinite(ref).all():
            assert np.all(np.abs(got.cpu().numpy() - ref) <= 1e-13 * (mag + np.abs(ref)) + 1e-300), name


@pytest.mark.parametrize("idx", range(int(DOUBLE["forest_count"])))
def test_double_precision_golden(ext, idx):
    p = "forest%02d_" % idx
    c = {k[len(p):]: DOUBLE[k] for k in DOUBLE.files if k.startswith(p)}
    check(ext, str(c["kind"]), c)


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_double_precision_against_the_reference_build(ext, kind):
    try:
        from oracle import build_ref
        ref = build_ref.load()
    except ImportError:
        pytest.skip("the reference build (oracle/_ref) is not here")
    gen = torch.Generator().manual_seed(77)
    B, C, T, depth, M = 300, 40, 17, 7, 3
    N = depth if kind == "fern" else 2 ** depth - 1
    x = torch.randn((B, C, 2), generator=gen, dtype=torch.float64)
    thr = torch.rand((T, N), generator=gen, dtype=torch.float64) * 6 - 3
    ord_ = torch.randint(0, C, (T, N), generator=gen)
    w = torch.randn((T, 2 ** depth, M), generator=gen, dtype=torch.float64)
    f = getattr(ref, kind + "_forward")(x, thr, ord_, w)
    g = torch.randn(f.shape, generator=gen, dtype=torch.float64)
    gx, gthr, _, gw = getattr(ref, kind + "_backward")(x, True, thr, True, ord_, False, w, True, g)
    margin, mord = getattr(ref, kind + "_marginmap")(x, thr, ord_, w)
    c = {"x": x.numpy(), "thr": thr.numpy(), "ord": ord_.numpy(), "w": w.numpy(), "g": g.numpy(), "out": f.numpy(),
         "gx": gx.numpy(), "gthr": gthr.numpy(), "gw": gw.numpy(), "margin": margin.numpy(), "margin_ord": mord.numpy(),
         "leaf": getattr(ref, kind + "_leafmap")(x, thr, ord_, w).numpy().astype(np.int64),
         "reach": getattr(ref, kind + "_reachability")(x, thr, ord_, w).numpy().astype(np.int64)}
    check(ext, kind, c)


def test_double_precision_modules(ext):
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(5)
    m = R.RandomHingeForest(12, 6, 4, extra_outputs=2).double().cuda()
    x = torch.randn(30, 12, dtype=torch.float64, device="cuda", requires_grad=True)
    y = m(x)
    assert y.dtype == torch.float64 and y.shape == (30, 6, 2)
    y.sum().backward()
    assert x.grad.dtype == torch.float64 and m.weights.grad.dtype == torch.float64
    conv = R.HingeTreeConv2d(2, 3, 2, 3).double().cuda()
    image = torch.randn(1, 2, 6, 6, dtype=torch.float64, device="cuda", requires_grad=True)
    out = conv(image)
    assert out.dtype == torch.float64
    out.sum().backward()
    assert image.grad.dtype == torch.float64 and conv.thresholds.grad.dtype == torch.float64
    with pytest.raises(ValueError):  # mixed precisions are refused, as in the reference
        ext.tree_forward(x.detach(), m.thresholds.detach().float(), m.ordinals, m.weights.detach())


# ---- the other operator families in double precision (tests/golden/families64.npz) ---------------------
# The reference instantiates every operator for float and double.  Forward results of the fixed-order kernels
# (fused linear, convolution, trie) equal the reference's CPU results bit for bit; fusion forward too; gradients are
# sums in free order and are held to 1e-12 of the largest entry of the reference's gradient (double precision leaves
# thirteen digits; the terms are O(1)).

FAMILIES64 = np.load(os.path.join(GOLDEN, "families64.npz"))


def family_case(prefix):
    n = len(prefix)
    return {k[n:]: FAMILIES64[k] for k in FAMILIES64.files if k.startswith(prefix)}


def close64(t, ref):
    ref = np.asarray(ref, dtype=np.float64)
    got = t.detach().cpu().numpy()
    return bool(np.all(np.abs(got - ref) <= 1e-12 * max(float(np.abs(ref).max()), 1e-300)))


@pytest.mark.parametrize("idx", range(int(FAMILIES64["linear_count"])))
def test_fused_linear_and_fusion_in_double(ext, idx):
    c = family_case("linear%02d_" % idx)
    kind = str(c["kind"])
    d = {k: dev(v) for k, v in c.items() if k != "kind"}
    assert d["x"].dtype == torch.float64
    if "vec" in d:
        out = getattr(ext, kind + "_fusion_fused_linear_forward")(d["x"], d["vec"], d["thr"], d["ord"], d["w"], d["lin"], d["bias"])
        grads = getattr(ext, kind + "_fusion_fused_linear_backward")(d["x"], True, d["vec"], True, d["thr"], True, d["ord"], False,
                                                                     d["w"], True, d["lin"], True, d["bias"], True, d["g"])
        names = ["gx", "gvec", "gthr", None, "gw", "glin", "gbias"]
        assert np.array_equal(getattr(ext, kind + "_fusion_forward")(d["x"], d["vec"], d["thr"], d["ord"], d["w"]).cpu().numpy(),
                              c["fusion_out"])
        fg = getattr(ext, kind + "_fusion_backward")(d["x"], True, d["vec"], True, d["thr"], True, d["ord"], False, d["w"], True,
                                                     d["fusion_g"])
        for got, name in zip((fg[0], fg[1], fg[2], fg[4]), ("fusion_gx", "fusion_gvec", "fusion_gthr", "fusion_gw")):
            assert close64(got, c[name]), name
    else:
        out = getattr(ext, kind + "_fused_linear_forward")(d["x"], d["thr"], d["ord"], d["w"], d["lin"], d["bias"])
        grads = getattr(ext, kind + "_fused_linear_backward")(d["x"], True, d["thr"], True, d["ord"], False, d["w"], True,
                                                              d["lin"], True, d["bias"], True, d["g"])
        names = ["gx", "gthr", None, "gw", "glin", "gbias"]
    assert out.dtype == torch.float64 and np.array_equal(out.cpu().numpy(), c["out"])
    for got, name in zip(grads, names):
        if name is not None:
            assert close64(got, c[name]), name


@pytest.mark.parametrize("idx", range(int(FAMILIES64["conv_count"])))
def test_convolution_in_double(ext, idx):
    c = family_case("conv%02d_" % idx)
    kind = str(c["kind"])
    geometry = [[int(v) for v in row] for row in c["geometry"]]
    dims = len(geometry[0])
    d = {k: dev(v) for k, v in c.items() if k not in ("kind", "geometry")}
    out = getattr(ext, "%s_conv%dd_forward" % (kind, dims))(d["x"], d["thr"], d["ord"], d["w"], *geometry)
    assert out.dtype == torch.float64 and np.array_equal(out.cpu().numpy(), c["out"])
    gx, gthr, _, gw = getattr(ext, "%s_conv%dd_backward" % (kind, dims))(d["x"], True, d["thr"], True, d["ord"], False, d["w"],
                                                                        True, d["g"], *geometry)
    assert close64(gx, c["gx"]) and close64(gthr, c["gthr"]) and close64(gw, c["gw"])


@pytest.mark.parametrize("idx", range(int(FAMILIES64["trie_count"])))
def test_trie_in_double(ext, idx):
    c = family_case("trie%02d_" % idx)
    d = {k: dev(v) for k, v in c.items()}
    out = ext.trie_forward(d["x"], d["thr"], d["ord"], d["w"])
    assert out.dtype == torch.float64 and np.array_equal(out.cpu().numpy(), c["out"])
    gx, gthr, _, gw = ext.trie_backward(d["x"], True, d["thr"], True, d["ord"], False, d["w"], True, d["g"])
    assert close64(gx, c["gx"]) and close64(gthr, c["gthr"]) and close64(gw, c["gw"])


def test_sparse_backward_in_double(ext):
    """Values and pattern of the sparse gradients against the dense double precision backward."""
    gen = torch.Generator().manual_seed(4)
    B, C, T, depth = 20, 9, 6, 4
    x = torch.randn(B, C, generator=gen, dtype=torch.float64).cuda()
    thr = (torch.rand(T, 2 ** depth - 1, generator=gen, dtype=torch.float64) * 4 - 2).cuda()
    ord_ = torch.randint(0, C, (T, 2 ** depth - 1), generator=gen).cuda()
    w = torch.randn(T, 2 ** depth, 2, generator=gen, dtype=torch.float64).cuda()
    g = torch.randn(B, T, 2, generator=gen, dtype=torch.float64).cuda()
    dense = ext.tree_backward(x, True, thr, True, ord_, False, w, True, g)
    sparse = ext.sparse_tree_backward(x, True, thr, True, ord_, False, w, True, g)
    for slot in (0, 1, 3):
        assert sparse[slot].is_sparse and sparse[slot].dtype == torch.float64
        assert close64(sparse[slot].to_dense(), dense[slot].cpu().numpy())
        assert int(sparse[slot]._nnz()) <= int((dense[slot] != 0).sum()) + int(sparse[slot]._nnz())  # pattern holds the non-zeros
        assert bool(((dense[slot] != 0) <= (sparse[slot].to_dense() != 0)).all())
