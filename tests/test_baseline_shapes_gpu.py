"""The five benchmark configurations at their full sizes.

Where the CPU oracle finishes in seconds (C1, C2, the forest stage of C5) the whole result is compared:
forward bit-exact, default backward within 1e-5 of the summed term magnitudes, fixed-order backward
bit-exact.  Where it does not (C3: 2^30 tree evaluations, C4: 2^31) the check is on properties that do not
depend on the size: rows / samples picked at random are bit-exact against the oracle, shards of the
batch concatenate to the whole (the multi-GPU decomposition), two runs give the same bits, per-tree
leaf counts add up to the batch, and parameter gradients are additive over batch shards.
"""
import numpy as np
import pytest
import torch

from conftest import random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cabi():
    from hingetreefortorch_b200 import _cabi
    _cabi.library()
    return _cabi


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


def equal(t, a):
    return np.array_equal(t.cpu().numpy(), a, equal_nan=True)


def grad_close(t, ref, scale):
    got = t.cpu().numpy().astype(np.float64)
    return np.all(np.abs(got - ref.astype(np.float64)) <= 1e-5 * scale + 1e-30)


def whole_forest_check(cabi, kind, x, thr, ord_, w, fixed_order=True):
    want = ho.forward(kind, x, thr, ord_, w)
    g = np.random.default_rng(3).standard_normal(want.shape).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    f = cabi.Forest(kind, dx, dw)
    assert equal(f.forward(dx, dthr, dord, dw), want)
    rx, rthr, rw = ho.backward(kind, x, thr, ord_, w, g)
    ax, athr, aw = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    assert grad_close(gx, rx, ax) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)
    if fixed_order:
        fd = cabi.Forest(kind, dx, dw, deterministic=True)
        for got, ref in zip(fd.backward(dx, dthr, dord, dw, dg), (rx, rthr, rw)):
            assert equal(got, ref)
    assert f.ordinal_flags() == 0


def test_c1_speedtest_shape_whole(cabi):
    x, thr, ord_, w = random_forest_inputs(1, "tree", 100, 1000, (), 100, 7, (1,))
    whole_forest_check(cabi, "tree", np.abs(x) % 1.0, thr, ord_, w)  # features in [0, 1) like torch.rand


def test_c2_fern_shape_whole(cabi):
    x, thr, ord_, w = random_forest_inputs(2, "fern", 4096, 256, (), 500, 10, (10,))
    whole_forest_check(cabi, "fern", x, thr, ord_, w)


def test_c5_forest_stage_whole(cabi):
    """8192 rows of 12700 normalised features, 100 trees of depth 7, tree j reads features 127 j .. 127 j + 126."""
    rng = np.random.default_rng(5)
    B, C, T, N = 8192, 12700, 100, 127
    x = rng.standard_normal((B, C)).astype(np.float32)
    thr = rng.uniform(-3, 3, (T, N)).astype(np.float32)
    ord_ = (np.arange(T * N, dtype=np.int64) % C).reshape(T, N)
    w = rng.standard_normal((T, 128)).astype(np.float32)
    whole_forest_check(cabi, "tree", x, thr, ord_, w)


def test_c3_inference_shape_properties(cabi):
    B, C, T, depth = 1048576, 128, 1024, 8
    _, thr, ord_, w = random_forest_inputs(3, "tree", 1, C, (), T, depth, ())
    gen = torch.Generator(device="cuda").manual_seed(33)
    dx = torch.randn((B, C), device="cuda", generator=gen)
    dthr, dord, dw = dev(thr, ord_, w)
    f = cabi.Forest("tree", dx, dw, backward_workspace=False)
    out = f.forward(dx, dthr, dord, dw)
    # random rows against the oracle
    rows = torch.from_numpy(np.sort(np.random.default_rng(0).choice(B, 256, replace=False))).cuda()
    assert equal(out[rows], ho.forward("tree", dx[rows].cpu().numpy(), thr, ord_, w))
    # the same bits again, and a checksum of per-row checksums that any changed element would move
    checksum = out.view(torch.int32).sum(dim=1, dtype=torch.int64).sum().item()
    again = f.forward(dx, dthr, dord, dw)
    assert again.view(torch.int32).sum(dim=1, dtype=torch.int64).sum().item() == checksum
    del again
    # batch shards (what each GPU of a multi-GPU run evaluates) concatenate to the whole
    for lo, hi in ((0, B // 8), (3 * (B // 8) + 5, 4 * (B // 8) + 77), (B - 1000, B)):
        part = dx[lo:hi].contiguous()
        shard = cabi.Forest("tree", part, dw, backward_workspace=False).forward(part, dthr, dord, dw)
        assert torch.equal(shard, out[lo:hi])
    # every row reaches exactly one leaf of every tree
    assert f.reachability(dx, dthr, dord).sum(dim=1).eq(B).all()
    assert f.ordinal_flags() == 0


def test_c4_convolution_shape_properties():
    from hingetreefortorch_b200 import _cabi
    B, Ci, Co, H, W, depth = 64, 64, 128, 64, 64, 5
    geometry = ((3, 3), (1, 1), (1, 1), (1, 1))
    rng = np.random.default_rng(6)
    thr = rng.uniform(-3, 3, (Co, Ci, 31)).astype(np.float32)
    ord_ = rng.integers(0, 9, (Co, Ci, 31)).astype(np.int64)
    w = rng.standard_normal((Co, Ci, 32)).astype(np.float32)
    gen = torch.Generator(device="cuda").manual_seed(66)
    dx = torch.randn((B, Ci, H, W), device="cuda", generator=gen)
    dg = torch.randn((B, Co, H, W), device="cuda", generator=gen)
    dthr, dord, dw = dev(thr, ord_, w)
    conv = _cabi.Conv("tree", dx, dw, *geometry)
    out = conv.forward(dx, dthr, dord, dw)
    assert torch.equal(out, conv.forward(dx, dthr, dord, dw))
    for b in (0, 37):  # single samples against the oracle, bit for bit
        assert equal(out[b:b + 1], ho.conv_forward("tree", dx[b:b + 1].cpu().numpy(), thr, ord_, w, *geometry))
    # batch shards
    half = dx[B // 2:].contiguous()
    assert torch.equal(_cabi.Conv("tree", half, dw, *geometry).forward(half, dthr, dord, dw), out[B // 2:])

    gx, gthr, gw = conv.backward(dx, dthr, dord, dw, dg)
    # the image gradient of a sample depends on that sample alone
    b = 37
    rx, rthr, rw = ho.conv_backward("tree", dx[b:b + 1].cpu().numpy(), thr, ord_, w, dg[b:b + 1].cpu().numpy(), *geometry)
    tol = 1e-4 * np.abs(rx).max()
    assert np.abs(gx[b:b + 1].cpu().numpy() - rx).max() <= tol
    # parameter gradients are sums over samples: the whole batch equals the sum of its shards
    parts = []
    for lo, hi in ((0, B // 2), (B // 2, B)):
        px, pg = dx[lo:hi].contiguous(), dg[lo:hi].contiguous()
        parts.append(_cabi.Conv("tree", px, dw, *geometry).backward(px, dthr, dord, dw, pg))
    for whole, a, c in ((gthr, parts[0][1], parts[1][1]), (gw, parts[0][2], parts[1][2])):
        scale = float(whole.abs().max())
        assert float((whole - (a + c)).abs().max()) <= 1e-4 * scale
    # and one sample's share of them against the oracle
    one = _cabi.Conv("tree", dx[b:b + 1].contiguous(), dw, *geometry).backward(
        dx[b:b + 1].contiguous(), dthr, dord, dw, dg[b:b + 1].contiguous())
    assert np.allclose(one[1].cpu().numpy(), rthr, rtol=1e-4, atol=1e-4 * np.abs(rthr).max())
    assert np.allclose(one[2].cpu().numpy(), rw, rtol=1e-4, atol=1e-4 * np.abs(rw).max())
    assert conv.status.item() == 0
