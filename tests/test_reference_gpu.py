"""This library beside the reference's own CUDA kernels on the same GPU and the same tensors.

The unmodified reference, built with its GPU translation units by `oracle/build_ref.py --gpu`
(hingetree_gpu.cu, hingetree_conv_gpu.cu, hingetree_fused_linear_gpu.cu), is a second checker
next to the CPU oracle: forward results have to be equal bit for bit (both compute
|margin| * weight with one rounding), maps equal, gradients within the usual bar.  Skipped where that
build is not present.  Batches stay far below 524 280 rows, the limit of the reference's launch
configuration (hingetree_gpu.cu:491-495).
"""
import os
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, grad_close, random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import build_ref
    try:
        return build_ref.load_gpu()
    except ImportError as e:
        pytest.skip(str(e))


@pytest.fixture(scope="module")
def ext():
    from hingetreefortorch_b200._ext import hingetree_cpp
    return hingetree_cpp


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


# (kind, B, C, inner, T, depth, extra): any-shape kernels, the tile kernel with the weights in its records,
# the tile kernel with several outputs per leaf, image-shaped input
SHAPES = [
    ("tree", 40, 12, (3,), 10, 4, (2,)),
    ("fern", 64, 20, (), 16, 6, ()),
    ("tree", 4096, 128, (), 64, 8, ()),
    ("fern", 2048, 64, (), 48, 10, (5,)),
    ("tree", 8, 16, (24, 24), 32, 5, ()),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "%s-B%d-T%d-d%d" % (s[0], s[1], s[4], s[5]))
def test_forward_and_maps_equal_the_reference_gpu_kernels(ref, ext, shape):
    kind = shape[0]
    x, thr, ord_, w = random_forest_inputs(5, *shape)
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    assert torch.equal(getattr(ext, kind + "_forward")(dx, dthr, dord, dw), getattr(ref, kind + "_forward")(dx, dthr, dord, dw))
    assert torch.equal(getattr(ext, kind + "_leafmap")(dx, dthr, dord, dw), getattr(ref, kind + "_leafmap")(dx, dthr, dord, dw))
    ours, theirs = getattr(ext, kind + "_marginmap")(dx, dthr, dord, dw), getattr(ref, kind + "_marginmap")(dx, dthr, dord, dw)
    assert torch.equal(ours[0], theirs[0]) and torch.equal(ours[1], theirs[1])
    assert torch.equal(getattr(ext, kind + "_reachability")(dx, dthr, dord, dw),
                       getattr(ref, kind + "_reachability")(dx, dthr, dord, dw))


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "%s-B%d-T%d-d%d" % (s[0], s[1], s[4], s[5]))
def test_backward_against_the_reference_gpu_kernels(ref, ext, shape):
    kind = shape[0]
    x, thr, ord_, w = random_forest_inputs(6, *shape)
    out_shape = (shape[1], shape[4]) + tuple(shape[3]) + tuple(shape[6])
    g = np.random.default_rng(1).standard_normal(out_shape).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    mags = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    for name in ("_backward", "_backward_deterministic"):
        ours = getattr(ext, kind + name)(dx, True, dthr, True, dord, False, dw, True, dg)
        theirs = getattr(ref, kind + name)(dx, True, dthr, True, dord, False, dw, True, dg)
        assert ours[2] is None and theirs[2] is None
        for slot, mag in zip((0, 1, 3), mags):
            # both sides sum in an order of their own: each is within 1e-5 * sum|terms| of the exact sum
            assert grad_close(ours[slot], theirs[slot].cpu().numpy(), mag, rel=2e-5), (name, slot)


CONV = [
    # x shape, Co, depth, extra, kernel, stride, padding, dilation
    ((2, 3, 6, 7), 4, 3, (), (3, 3), (1, 1), (1, 1), (1, 1)),
    ((1, 2, 8, 9), 3, 2, (2,), (2, 3), (2, 1), (1, 2), (2, 1)),
    ((2, 20, 48, 70), 8, 5, (), (3, 3), (1, 1), (1, 1), (1, 1)),  # the shared-memory tile kernels
]


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("case", CONV, ids=[str(c[0]) for c in CONV])
def test_convolution_against_the_reference_gpu_kernels(ref, ext, kind, case):
    """The reference adds the input channels in ascending order with one launch per (sample, channel)
    (hingetree_conv_gpu.cu:368-380), as its CPU loop does, but nvcc contracts its `out += |margin| * w` into a
    fused multiply-add, which the CPU build (the oracle this library equals bit for bit) does not have: the
    forward agrees to a rounding per term; the backward scatters with atomics."""
    xs, Co, depth, extra, kernel, stride, padding, dilation = case
    rng = np.random.default_rng(CONV.index(case))
    Ci, N, cells = xs[1], (2 ** depth - 1 if kind == "tree" else depth), int(np.prod(kernel))
    x = rng.standard_normal(xs).astype(np.float32)
    thr = rng.uniform(-1, 1, (Co, Ci, N)).astype(np.float32)
    ord_ = rng.integers(0, cells, (Co, Ci, N)).astype(np.int64)
    w = rng.standard_normal((Co, Ci, 2 ** depth) + extra).astype(np.float32)
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    geometry = [list(kernel), list(stride), list(padding), list(dilation)]
    ours = getattr(ext, kind + "_conv2d_forward")(dx, dthr, dord, dw, *geometry)
    theirs = getattr(ref, kind + "_conv2d_forward")(dx, dthr, dord, dw, *geometry)
    terms = ho.conv_forward(kind, x, thr, ord_, np.abs(w), kernel, stride, padding, dilation)  # sum of |margin| * |w|
    assert grad_close(ours, theirs.cpu().numpy(), terms, rel=2e-6)
    g = rng.standard_normal(tuple(ours.shape)).astype(np.float32)
    dg, = dev(g)
    mags = ho.magnitudes(ho.conv_backward, kind, x, thr, ord_, w, g, kernel, stride, padding, dilation)
    a = getattr(ext, kind + "_conv2d_backward")(dx, True, dthr, True, dord, False, dw, True, dg, *geometry)
    b = getattr(ref, kind + "_conv2d_backward")(dx, True, dthr, True, dord, False, dw, True, dg, *geometry)
    for slot, mag in zip((0, 1, 3), mags):
        assert grad_close(a[slot], b[slot].cpu().numpy(), mag, rel=2e-5), slot


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_fused_linear_against_the_reference_gpu_kernels(ref, ext, kind):
    """The reference's fused forward adds into the output with atomics (hingetree_fused_linear_gpu.cu:73-108),
    so the comparison is at the bar of a sum in free order on both sides."""
    B, C, T, depth, O = 96, 24, 20, 5, 7
    x, thr, ord_, w = random_forest_inputs(9, kind, B, C, (), T, depth, ())
    rng = np.random.default_rng(2)
    lin = rng.standard_normal((O, T)).astype(np.float32)
    bias = rng.standard_normal((O,)).astype(np.float32)
    g = rng.standard_normal((B, O)).astype(np.float32)
    dx, dthr, dord, dw, dlin, dbias, dg = dev(x, thr, ord_, w, lin, bias, g)
    ours = getattr(ext, kind + "_fused_linear_forward")(dx, dthr, dord, dw, dlin, dbias)
    theirs = getattr(ref, kind + "_fused_linear_forward")(dx, dthr, dord, dw, dlin, dbias)
    terms = np.abs(ho.forward(kind, x, thr, ord_, w)) @ np.abs(lin).T + np.abs(bias)  # sum of |terms| per output
    assert grad_close(ours, theirs.cpu().numpy(), terms, rel=2e-5)
    a = getattr(ext, kind + "_fused_linear_backward")(dx, True, dthr, True, dord, False, dw, True, dlin, True, dbias, True, dg)
    b = getattr(ref, kind + "_fused_linear_backward")(dx, True, dthr, True, dord, False, dw, True, dlin, True, dbias, True, dg)
    mags = ho.magnitudes(ho.linear_backward, kind, x, thr, ord_, w, lin, g)
    for slot, mag in zip((0, 1, 3, 4, 5), mags):
        assert grad_close(a[slot], b[slot].cpu().numpy(), mag, rel=2e-5), slot
