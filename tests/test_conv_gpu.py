"""Convolutional hinge trees / ferns and contract / expand on a GPU, against the CPU oracle.

Bars: the convolution forward is bit-exact (input channels are added in the reference's order);
its gradients (summation order is free) match within 1e-5 of the summed term magnitudes; contract and
expand move bytes and are exact for every element type, and expand(contract(x)) == x whenever the
windows tile the image without padding.
"""
import numpy as np
import pytest
import torch

from conftest import grad_close
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


CONV_CASES = [
    # dims, x shape, Co, depth, extra, kernel, stride, padding, dilation
    (1, (2, 3, 9), 4, 2, (), (3,), (1,), (1,), (1,)),
    (1, (2, 2, 40), 3, 3, (2,), (5,), (2,), (0,), (2,)),
    (2, (2, 3, 6, 7), 4, 3, (), (3, 3), (1, 1), (1, 1), (1, 1)),
    (2, (1, 2, 16, 17), 5, 5, (), (3, 3), (1, 1), (1, 1), (1, 1)),
    (2, (1, 2, 8, 9), 3, 2, (2,), (2, 3), (2, 1), (1, 2), (2, 1)),
    (2, (3, 4, 12, 12), 6, 4, (9,), (3, 3), (2, 2), (0, 0), (1, 1)),
    (3, (1, 2, 5, 6, 4), 2, 2, (), (2, 3, 2), (1, 2, 1), (1, 0, 1), (1, 1, 2)),
    # large enough for the shared-memory tile kernel (one output per leaf, >= 2^20 tree evaluations):
    # ragged channel chunks and output-channel blocks, few tiles (output channels split over CTAs)
    (2, (2, 20, 48, 70), 8, 5, (), (3, 3), (1, 1), (1, 1), (1, 1)),
    # stride, dilation, padding wider than the window overhang, non-square window, odd channel counts
    (2, (1, 7, 67, 90), 50, 4, (), (3, 5), (2, 1), (2, 3), (2, 1)),
    # window offsets beyond one byte
    (2, (1, 4, 60, 64), 80, 3, (), (3, 3), (1, 1), (6, 6), (6, 6)),
    # 1-D: one tile row
    (1, (4, 6, 3000), 16, 6, (), (7,), (1,), (3,), (1,)),
    # depth 7: the parameter kernel with 4 columns per bin (8 lane groups); depth 8: beyond it, the image-gradient
    # kernel collects the parameter gradients in its shared bins as well
    (2, (2, 8, 48, 64), 24, 7, (), (3, 3), (1, 1), (1, 1), (1, 1)),
    (2, (2, 8, 48, 64), 24, 8, (), (3, 3), (1, 1), (1, 1), (1, 1)),
]


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("case", CONV_CASES, ids=[str(c[:2]) for c in CONV_CASES])
def test_convolution_matches_oracle(kind, case):
    from hingetreefortorch_b200 import _cabi
    dims, xs, Co, depth, extra, kernel, stride, padding, dilation = case
    rng = np.random.default_rng(CONV_CASES.index(case))
    Ci, N, cells = xs[1], (2 ** depth - 1 if kind == "tree" else depth), int(np.prod(kernel))
    x = rng.standard_normal(xs).astype(np.float32)
    thr = rng.uniform(-1, 1, (Co, Ci, N)).astype(np.float32)
    ord_ = rng.integers(0, cells, (Co, Ci, N)).astype(np.int64)
    w = rng.standard_normal((Co, Ci, 2 ** depth) + extra).astype(np.float32)
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    conv = _cabi.Conv(kind, dx, dw, kernel, stride, padding, dilation)
    out = conv.forward(dx, dthr, dord, dw)
    want = ho.conv_forward(kind, x, thr, ord_, w, kernel, stride, padding, dilation)
    assert out.shape == want.shape and np.array_equal(out.cpu().numpy(), want)
    g = rng.standard_normal(want.shape).astype(np.float32)
    dg, = dev(g)
    gx, gthr, gw = conv.backward(dx, dthr, dord, dw, dg)
    rx, rthr, rw = ho.conv_backward(kind, x, thr, ord_, w, g, kernel, stride, padding, dilation)
    ax, athr, aw = ho.magnitudes(ho.conv_backward, kind, x, thr, ord_, w, g, kernel, stride, padding, dilation)
    assert grad_close(gx, rx, ax) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)
    assert conv.status.item() == 0


def test_convolution_equals_sum_of_plain_forests_on_unfolded_channels():
    """The identity the reference's design rests on: conv2d == sum over channels of a forest on im2col patches."""
    from hingetreefortorch_b200 import _cabi
    rng = np.random.default_rng(5)
    B, Ci, Co, depth, H, W = 2, 3, 4, 3, 7, 6
    x = rng.standard_normal((B, Ci, H, W)).astype(np.float32)
    thr = rng.uniform(-1, 1, (Co, Ci, 7)).astype(np.float32)
    ord_ = rng.integers(0, 9, (Co, Ci, 7)).astype(np.int64)
    w = rng.standard_normal((Co, Ci, 8)).astype(np.float32)
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    out = _cabi.Conv("tree", dx, dw, (3, 3), (1, 1), (1, 1), (1, 1)).forward(dx, dthr, dord, dw)
    total = torch.zeros_like(out)
    for c in range(Ci):
        patches = torch.nn.functional.unfold(dx[:, c:c + 1], 3, padding=1).contiguous()  # [B, 9, H*W]
        tw = dw[:, c].contiguous()
        forest = _cabi.Forest("tree", patches, tw)
        total += forest.forward(patches, dthr[:, c].contiguous(), dord[:, c].contiguous(), tw).view_as(out)
    assert torch.equal(out, total)


@pytest.mark.parametrize("dtype", [torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.float32,
                                   torch.float64])
def test_contract_expand_every_dtype(dtype):
    from hingetreefortorch_b200 import _cabi
    for xs, window, padding in [((2, 3, 7, 9), (2, 3), (1, 0)), ((1, 2, 8, 8), (4, 4), (2, 2)),
                                ((1, 2, 5, 6, 7), (2, 3, 2), (1, 1, 0)), ((2, 1, 6, 6), (3, 3), (0, 0))]:
        x = (torch.rand(xs) * 100).to(dtype)
        c = _cabi.contract(x.cuda(), window, padding)
        want = ho.contract(x.numpy(), window, padding)
        assert np.array_equal(c.cpu().numpy(), want)
        e = _cabi.expand(c, padding)
        assert np.array_equal(e.cpu().numpy(), ho.expand(want, padding))
        if not any(padding) and all(s % w == 0 for s, w in zip(xs[2:], window)):
            assert torch.equal(e.cpu(), x)  # round trip


def test_conv_modules_and_contract_expand_autograd():
    from hingetreefortorch_b200 import RandomHingeForest as R, HingeTree as F
    torch.manual_seed(2)
    m = R.HingeTreeConv2d(3, 5, 4, 3, padding=1).cuda()
    x = torch.randn(2, 3, 10, 11, device="cuda", requires_grad=True)
    y = m(x)
    assert y.shape == (2, 5, 10, 11)
    y.sum().backward()
    want = ho.conv_forward("tree", x.detach().cpu().numpy(), m.thresholds.detach().cpu().numpy(), m.ordinals.cpu().numpy(),
                           m.weights.detach().cpu().numpy(), (3, 3), (1, 1), (1, 1), (1, 1))
    assert np.array_equal(y.detach().cpu().numpy(), want)
    assert x.grad is not None and m.thresholds.grad.shape == m.thresholds.shape
    f3 = R.HingeFernConv3d(2, 3, 3, 2, extra_outputs=4).cuda()
    assert f3(torch.randn(1, 2, 4, 5, 6, device="cuda")).shape == (1, 3, 3, 4, 5, 4)
    assert R.HingeTreeConv1d(2, 3, 2, 3, stride=2).cuda()(torch.randn(2, 2, 9, device="cuda")).shape == (2, 3, 4)

    img = torch.randn(2, 3, 8, 8, device="cuda", requires_grad=True)
    patches = F.Contract(4)(img)
    assert patches.shape == (2, 3, 2, 2, 4, 4)
    back = F.Expand()(patches)
    assert torch.equal(back, img)
    back.sum().backward()
    assert torch.equal(img.grad, torch.ones_like(img))
    with pytest.raises(ValueError):
        F.contract(img.detach(), [9, 9], [0, 0])  # window larger than the image
