"""The five benchmark configurations at their full sizes.

Where the CPU oracle finishes in seconds (C1, C2, the forest stage of C5) the whole result is compared:
forward bit-exact, default backward within 1e-5 of the summed term magnitudes, fixed-order backward
bit-exact.  Where it does not (C3: 2^30 tree evaluations, C4: 2^31) the check is on properties that do not
depend on the size: rows / samples picked at random are bit-exact against the oracle, shards of the
batch concatenate to the whole (the multi-GPU decomposition), two runs give the same bits, per-tree
leaf counts add up to the batch, and parameter gradients are additive over batch shards.
"""
import os

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


def test_c3_backward_shape_properties(cabi):
    """Forward + backward of the large-batch configuration (the benchmark's fwd_bwd figure) at full size.
    The x gradient of a row depends on that row alone and is added in tree order in both modes: sampled
    rows are bit-exact against the oracle.  Parameter gradients are sums over rows: the whole batch
    equals the sum of two batch shards within 1e-5 of the summed term magnitudes, and one shard small
    enough for the oracle matches it at the same bar."""
    B, C, T, depth = 1048576, 128, 1024, 8
    _, thr, ord_, w = random_forest_inputs(3, "tree", 1, C, (), T, depth, ())
    gen = torch.Generator(device="cuda").manual_seed(34)
    dx = torch.randn((B, C), device="cuda", generator=gen)
    dg = torch.randn((B, T), device="cuda", generator=gen)
    dthr, dord, dw = dev(thr, ord_, w)
    f = cabi.Forest("tree", dx, dw)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    assert f.ordinal_flags() == 0
    rows = np.sort(np.random.default_rng(1).choice(B, 64, replace=False))
    drows = torch.from_numpy(rows).cuda()
    xs, gs = dx[drows].cpu().numpy(), dg[drows].cpu().numpy()
    rx, _, _ = ho.backward("tree", xs, thr, ord_, w, gs)
    assert equal(gx[drows], rx)
    # a shard the oracle can follow: 2048 rows, all three gradients
    n = 2048
    px, pg = dx[:n].contiguous(), dg[:n].contiguous()
    part = cabi.Forest("tree", px, dw).backward(px, dthr, dord, dw, pg)
    want = ho.backward("tree", px.cpu().numpy(), thr, ord_, w, pg.cpu().numpy())
    mags = ho.backward_magnitudes("tree", px.cpu().numpy(), thr, ord_, w, pg.cpu().numpy())
    for got, ref, mag in zip(part, want, mags):
        assert grad_close(got, ref, mag)
    # additivity over 16 batch shards.  The scale is rigorous: the sum over shards of |shard gradient| never
    # exceeds the summed term magnitudes, so this bar is at least as strict as the stated one.
    shards = 16
    total = [np.zeros(thr.shape), np.zeros(w.shape)]
    scale = [np.zeros(thr.shape), np.zeros(w.shape)]
    for k in range(shards):
        lo, hi = k * (B // shards), (k + 1) * (B // shards)
        hx, hg = dx[lo:hi].contiguous(), dg[lo:hi].contiguous()
        part = cabi.Forest("tree", hx, dw).backward(hx, dthr, dord, dw, hg)
        assert torch.equal(part[0], gx[lo:hi])
        for acc, mag, t in zip(total, scale, part[1:]):
            t = t.cpu().numpy().astype(np.float64)
            acc += t
            mag += np.abs(t)
    assert grad_close(gthr, total[0], scale[0]) and grad_close(gw, total[1], scale[1])


def test_trained_forest_of_the_reference_example(cabi):
    """Trained parameters instead of random ones: the forests of the reference's renal-cell-carcinoma
    example (100 trees of depth 7 over 100 channels, 8 x 8 outputs per leaf) on its input shape
    x [8, 100, 32, 32].  The parameters are read from oracle/_ref/trained_forests.npz, which
    oracle/build_ref.py extracts from a checkout of the reference; skipped where that file is absent."""
    from oracle import build_ref
    if not os.path.exists(build_ref.trained_forest_path()):
        pytest.skip("no trained parameters: run python oracle/build_ref.py --reference <checkout>")
    data = np.load(build_ref.trained_forest_path())
    for n in range(int(data["count"])):
        thr, ord_, w = data["thr%d" % n], data["ord%d" % n], data["w%d" % n]
        assert thr.shape == (100, 127) and w.shape == (100, 128, 8, 8) and ord_.min() >= 0 and ord_.max() < 100
        rng = np.random.default_rng(40 + n)
        x = (3.0 * rng.standard_normal((8, 100, 32, 32))).astype(np.float32)
        want = ho.forward("tree", x, thr, ord_, w)
        g = rng.standard_normal(want.shape).astype(np.float32)
        dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
        f = cabi.Forest("tree", dx, dw)
        assert equal(f.forward(dx, dthr, dord, dw), want)
        leaf = ho.maps("tree", x, thr, ord_, w)[0]
        assert equal(f.leafmap(dx, dthr, dord), leaf)
        ref = ho.backward("tree", x, thr, ord_, w, g)
        mags = ho.backward_magnitudes("tree", x, thr, ord_, w, g)
        for got, r, m in zip(f.backward(dx, dthr, dord, dw, dg), ref, mags):
            assert grad_close(got, r, m)
        fd = cabi.Forest("tree", dx, dw, deterministic=True)
        for got, r in zip(fd.backward(dx, dthr, dord, dw, dg), ref):
            assert equal(got, r)
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
    one_x, one_g = dx[b:b + 1].cpu().numpy(), dg[b:b + 1].cpu().numpy()
    rx, rthr, rw = ho.conv_backward("tree", one_x, thr, ord_, w, one_g, *geometry)
    ax, athr, aw = ho.magnitudes(ho.conv_backward, "tree", one_x, thr, ord_, w, one_g, *geometry)
    assert grad_close(gx[b:b + 1], rx, ax)  # 1e-5 of the summed term magnitudes, per pixel
    # parameter gradients are sums over samples: the whole batch equals the sum of its 64 single-sample
    # gradients.  The scale is rigorous: the sum over samples of |sample gradient| never exceeds the summed
    # term magnitudes, so this bar is at least as strict as the stated one.
    total = [np.zeros(thr.shape), np.zeros(w.shape)]
    scale = [np.zeros(thr.shape), np.zeros(w.shape)]
    for s_ in range(B):
        px, pg = dx[s_:s_ + 1].contiguous(), dg[s_:s_ + 1].contiguous()
        part = _cabi.Conv("tree", px, dw, *geometry).backward(px, dthr, dord, dw, pg)
        for acc, mag, t in zip(total, scale, part[1:]):
            t = t.cpu().numpy().astype(np.float64)
            acc += t
            mag += np.abs(t)
    assert grad_close(gthr, total[0], scale[0]) and grad_close(gw, total[1], scale[1])
    # and one sample's share of them against the oracle
    one = _cabi.Conv("tree", dx[b:b + 1].contiguous(), dw, *geometry).backward(
        dx[b:b + 1].contiguous(), dthr, dord, dw, dg[b:b + 1].contiguous())
    assert grad_close(one[1], rthr, athr) and grad_close(one[2], rw, aw)
    assert conv.status.item() == 0
