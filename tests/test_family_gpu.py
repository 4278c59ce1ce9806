"""Image+vector fusion forests and forests followed by a linear layer, against the CPU oracle.

Bars: the fusion forward and the fused-linear forward are bit-exact (the fused-linear forward adds
its terms in the reference CPU order); gradients match within 1e-5 of the summed term magnitudes
(these backwards scatter with atomics, so their summation order is free)."""
import numpy as np
import pytest
import torch

from conftest import grad_close, random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu


def dev(*arrays):
    return [None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


CASES = [
    # kind, B, C, inner, T, depth, extra, O, Cv
    ("tree", 64, 12, (), 10, 4, (), 5, 0),
    ("fern", 33, 9, (3,), 7, 5, (2,), 4, 0),
    ("tree", 40, 6, (2, 2), 9, 3, (2,), 3, 5),
    ("fern", 50, 8, (), 11, 6, (), 6, 4),
    ("tree", 257, 20, (), 33, 7, (), 10, 0),
]


@pytest.mark.parametrize("case", CASES, ids=[str(c) for c in CASES])
def test_fused_linear_and_fusion(case):
    from hingetreefortorch_b200 import _cabi
    kind, B, C, inner, T, depth, extra, O, Cv = case
    rng = np.random.default_rng(CASES.index(case))
    x, thr, ord_, w = random_forest_inputs(50 + CASES.index(case), kind, B, C, inner, T, depth, extra)
    vec = rng.standard_normal((B, Cv)).astype(np.float32) if Cv else None
    if Cv:
        ord_ = rng.integers(0, C + Cv, ord_.shape).astype(np.int64)
    lin = rng.standard_normal((O, T)).astype(np.float32)
    bias = rng.standard_normal(O).astype(np.float32)
    dx, dvec, dthr, dord, dw, dlin, dbias = dev(x, vec, thr, ord_, w, lin, bias)
    fam = _cabi.ForestFamily(kind, dx, dw, vec=dvec, lin=dlin)

    out = fam.linear_forward(dx, dvec, dthr, dord, dw, dlin, dbias)
    want = ho.linear_forward(kind, x, thr, ord_, w, lin, bias, vec=vec)
    assert out.shape == want.shape and np.array_equal(out.cpu().numpy(), want)
    g = rng.standard_normal(want.shape).astype(np.float32)
    dg, = dev(g)
    gx, gvec, gthr, gw, glin = fam.linear_backward(dx, dvec, dthr, dord, dw, dlin, dg)
    ref = ho.linear_backward(kind, x, thr, ord_, w, lin, g, vec=vec)
    mag = ho.magnitudes(ho.linear_backward, kind, x, thr, ord_, w, lin, g, vec=vec)
    if Cv:
        rx, rvec, rthr, rw, rlin, _ = ref
        ax, avec, athr, aw, alin, _ = mag
        assert grad_close(gvec, rvec, avec)
    else:
        rx, rthr, rw, rlin, _ = ref
        ax, athr, aw, alin, _ = mag
    assert grad_close(gx, rx, ax) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw) and grad_close(glin, rlin, alin)
    assert fam.status.item() == 0

    if Cv:
        plain = _cabi.ForestFamily(kind, dx, dw, vec=dvec)
        out = plain.fusion_forward(dx, dvec, dthr, dord, dw)
        want = ho.forward(kind, x, thr, ord_, w, vec=vec)
        assert np.array_equal(out.cpu().numpy(), want)
        g2 = rng.standard_normal(want.shape).astype(np.float32)
        dg2, = dev(g2)
        gimg, gvec, gthr, gw = plain.fusion_backward(dx, dvec, dthr, dord, dw, dg2)
        rimg, rvec, rthr, rw = ho.backward(kind, x, thr, ord_, w, g2, vec=vec)
        aimg, avec, athr, aw = ho.magnitudes(ho.backward, kind, x, thr, ord_, w, g2, vec=vec)
        assert grad_close(gimg, rimg, aimg) and grad_close(gvec, rvec, avec)
        assert grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)


def test_modules_fused_linear_and_fusion():
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(1)
    m = R.RandomHingeForestFusedLinear(16, 12, 5, 4, extra_outputs=2).cuda()
    x = torch.randn(32, 16, device="cuda", requires_grad=True)
    y = m(x)
    assert y.shape == (32, 5, 2)
    y.square().sum().backward()
    args = [t.detach().cpu().numpy() for t in (x, m.thresholds, m.ordinals, m.weights, m.linear_weights, m.linear_bias)]
    assert np.array_equal(y.detach().cpu().numpy(), ho.linear_forward("tree", *args))
    g = (2 * y).detach().cpu().numpy()
    gx, gthr, gw, glin, gbias = ho.linear_backward("tree", args[0], args[1], args[2], args[3], args[4], g)
    ax, athr, aw, alin, abias = ho.magnitudes(ho.linear_backward, "tree", args[0], args[1], args[2], args[3], args[4], g)
    assert grad_close(x.grad, gx, ax) and grad_close(m.thresholds.grad, gthr, athr) and grad_close(m.weights.grad, gw, aw)
    assert grad_close(m.linear_weights.grad, glin, alin) and grad_close(m.linear_bias.grad, gbias, abias)

    f = R.RandomHingeFernFusion(6, 3, 8, 4).cuda()
    img = torch.randn(5, 6, 4, 4, device="cuda", requires_grad=True)
    vec = torch.randn(5, 3, device="cuda", requires_grad=True)
    y = f(img, vec)
    assert y.shape == (5, 8, 4, 4)
    y.sum().backward()
    want = ho.forward("fern", img.detach().cpu().numpy(), f.thresholds.detach().cpu().numpy(), f.ordinals.cpu().numpy(),
                      f.weights.detach().cpu().numpy(), vec=vec.detach().cpu().numpy())
    assert np.array_equal(y.detach().cpu().numpy(), want)
    assert img.grad is not None and vec.grad is not None and vec.grad.shape == (5, 3)

    ff = R.RandomHingeForestFusionFusedLinear(6, 3, 8, 2, 3).cuda()
    y = ff(img.detach(), vec.detach().requires_grad_(True))
    assert y.shape == (5, 2, 4, 4)
    y.sum().backward()
