"""Parity of the CUDA path with the CPU oracle, called through the C ABI (ctypes), on the
golden vectors of the reference and on seeded synthetic inputs.

Bars: forward, leaf map, margin map and reachability are bit-exact.  The default backward
matches within rtol 1e-5 of the per-element term magnitude (its summation order is free);
the deterministic backward is bit-exact against the oracle, whose loops are the reference
CPU loops, and identical from run to run.
"""
import numpy as np
import pytest
import torch

from conftest import forest_case, forest_case_ids, random_forest_inputs
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
    """|t - ref| <= 1e-5 * scale, scale = sum of |terms| that went into each element."""
    got = t.cpu().numpy().astype(np.float64)
    return np.all(np.abs(got - ref.astype(np.float64)) <= 1e-5 * scale + 1e-30)


def check_case(cabi, kind, x, thr, ord_, w, g, expect=None):
    if expect is None:
        leaf, margin, mord, reach = ho.maps(kind, x, thr, ord_, w)
        gx, gthr, gw = ho.backward(kind, x, thr, ord_, w, g)
        expect = dict(out=ho.forward(kind, x, thr, ord_, w), leaf=leaf, margin=margin, margin_ord=mord, reach=reach,
                      gx=gx, gthr=gthr, gw=gw)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    f = cabi.Forest(kind, dx, dw)
    assert equal(f.forward(dx, dthr, dord, dw), expect["out"])
    assert equal(f.leafmap(dx, dthr, dord), expect["leaf"])
    margin, mord = f.marginmap(dx, dthr, dord)
    assert equal(margin, expect["margin"]) and equal(mord, expect["margin_ord"])
    assert equal(f.reachability(dx, dthr, dord), expect["reach"])
    assert f.ordinal_flags() == 0

    # magnitude of what was summed into each gradient element (for the tolerance)
    ax, athr, aw = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    finite = np.isfinite(expect["gx"]).all() and np.isfinite(expect["gthr"]).all() and np.isfinite(expect["gw"]).all()
    if finite:
        assert grad_close(gx, expect["gx"], ax)
        assert grad_close(gthr, expect["gthr"], athr)
        assert grad_close(gw, expect["gw"], aw)

    fd = cabi.Forest(kind, dx, dw, deterministic=True)
    first = fd.backward(dx, dthr, dord, dw, dg)
    for t, name in zip(first, ("gx", "gthr", "gw")):
        assert equal(t, expect[name]), name
    second = fd.backward(dx, dthr, dord, dw, dg)
    for a, b in zip(first, second):
        assert torch.equal(a, b) or (torch.isnan(a) == torch.isnan(b)).all()


@pytest.mark.parametrize("idx", forest_case_ids())
def test_golden_vectors_of_the_reference(cabi, golden_forest, idx):
    c = forest_case(golden_forest, idx)
    check_case(cabi, c["kind"], c["x"], c["thr"], c["ord"], c["w"], c["g"], expect=c)


SHAPES = [
    # B, C, inner, T, depth, extra
    (1, 1, (), 1, 1, ()),
    (31, 9, (), 7, 2, ()),
    (32, 128, (), 8, 8, ()),
    (33, 256, (), 9, 5, (1,)),
    (100, 1000, (), 100, 7, (1,)),
    (257, 128, (), 65, 8, ()),
    (64, 16, (), 33, 10, (10,)),
    (5, 3, (17,), 6, 3, (2,)),
    (2, 7, (8, 8), 5, 4, (2, 2)),
    (3, 5, (3,), 4, 12, ()),
]


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", SHAPES, ids=[str(s) for s in SHAPES])
def test_synthetic_shapes(cabi, kind, shape):
    B, C, inner, T, depth, extra = shape
    x, thr, ord_, w = random_forest_inputs(2 * SHAPES.index(shape) + (kind == "fern"), kind, B, C, inner, T, depth, extra)
    g = np.random.default_rng(1).standard_normal((B, T) + inner + extra).astype(np.float32)
    check_case(cabi, kind, x, thr, ord_, w, g)


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_ties_zero_margins_and_hot_ordinals(cabi, kind):
    # quantised values give exact ties and exact zeros; all ordinals on two features makes every
    # sample of a tree hit the same gradient elements
    x, thr, ord_, w = random_forest_inputs(5, kind, 200, 6, (), 12, 6, (3,), quantise=True)
    ord_ = ord_ % 2
    g = np.random.default_rng(2).standard_normal((200, 12, 3)).astype(np.float32)
    check_case(cabi, kind, x, thr, ord_, w, g)


def test_fern_depth_20(cabi):
    x, thr, ord_, w = random_forest_inputs(9, "fern", 50, 40, (), 2, 20, ())
    g = np.ones((50, 2), np.float32)
    check_case(cabi, "fern", x, thr, ord_, w, g)


def test_empty_batch_and_no_trees(cabi):
    for (B, T) in [(0, 4), (3, 0)]:
        x, thr, ord_, w = random_forest_inputs(1, "tree", B, 5, (), T, 3, ())
        dx, dthr, dord, dw = dev(x, thr, ord_, w)
        f = cabi.Forest("tree", dx, dw)
        assert tuple(f.forward(dx, dthr, dord, dw).shape) == (B, T)
        gx, gthr, gw = f.backward(dx, dthr, dord, dw, torch.zeros(B, T, device="cuda"))
        assert float(gx.abs().sum()) == 0 and float(gthr.abs().sum()) == 0 and float(gw.abs().sum()) == 0


def test_out_of_range_ordinals_are_flagged_and_never_dereferenced(cabi):
    x, thr, ord_, w = random_forest_inputs(3, "tree", 16, 8, (), 4, 3, ())
    bad = ord_.copy()
    bad[1, 2] = 8
    bad[2, 0] = -1
    dx, dthr, dord, dw = dev(x, thr, bad, w)
    f = cabi.Forest("tree", dx, dw)
    out = f.forward(dx, dthr, dord, dw)
    assert f.ordinal_flags() & cabi.HT_FLAG_ORDINAL_RANGE
    # the offending ordinals were read as 0: same result as the clamped parameters
    clamped = bad.copy()
    clamped[1, 2] = 0
    clamped[2, 0] = 0
    assert equal(out, ho.forward("tree", x, thr, clamped, w))


def test_workspace_is_checked(cabi):
    import ctypes
    x, thr, ord_, w = random_forest_inputs(3, "tree", 4, 8, (), 4, 3, ())
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    f = cabi.Forest("tree", dx, dw)
    out = torch.empty(4, 4, device="cuda")
    lib = cabi.library()
    args = (ctypes.byref(f.problem), cabi._ptr(dx), cabi._ptr(dthr), cabi._ptr(dord), cabi._ptr(dw), cabi._ptr(out))
    rc = lib.ht_forest_forward_f32(*args, cabi._ptr(f.workspace), ctypes.c_size_t(8), cabi._ptr(f.status), None)
    assert rc == -4
    rc = lib.ht_forest_forward_f32(*args, ctypes.c_void_p(f.workspace.data_ptr() + 4), ctypes.c_size_t(1 << 20),
                                   cabi._ptr(f.status), None)
    assert rc == -4


def test_large_batch_properties(cabi):
    """At a size the oracle cannot finish quickly: a random slice is bit-exact, shards concatenate to
    the whole (the multi-GPU decomposition), and reachability sums to the number of positions."""
    B, C, T, depth = 65536, 128, 256, 8
    x, thr, ord_, w = random_forest_inputs(11, "tree", B, C, (), T, depth, ())
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    f = cabi.Forest("tree", dx, dw)
    out = f.forward(dx, dthr, dord, dw)
    rows = np.random.default_rng(0).choice(B, 64, replace=False)
    assert np.array_equal(out[torch.from_numpy(rows).cuda()].cpu().numpy(), ho.forward("tree", x[rows], thr, ord_, w))
    halves = []
    for part in (dx[: B // 2].contiguous(), dx[B // 2:].contiguous()):
        halves.append(cabi.Forest("tree", part, dw).forward(part, dthr, dord, dw))
    assert torch.equal(torch.cat(halves), out)
    reach = f.reachability(dx, dthr, dord)
    assert reach.sum(dim=1).eq(B).all()
    leaf = f.leafmap(dx, dthr, dord)
    counts = torch.zeros_like(reach).scatter_add_(1, leaf.t().contiguous(), torch.ones(T, B, dtype=torch.int64, device="cuda"))
    assert torch.equal(counts, reach)


TILED_SHAPES = [
    # B, C, T, depth: large enough for the shared-memory tile kernel (tabular input, one output per leaf)
    (1000, 128, 40, 8),
    (513, 64, 70, 5),
    (300, 300, 129, 7),   # more than 256 features: 16-bit compact ordinals
    (257, 1000, 132, 7),  # wide rows: small sample tiles
    (4096, 16, 9, 10),
    (2048, 32, 17, 1),
    (600, 32, 70, 11),    # deep trees: one or two trees per warp at a time
    (3000, 24, 13, 9),
]


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", TILED_SHAPES, ids=[str(s) for s in TILED_SHAPES])
def test_tile_kernel_shapes_with_special_values(cabi, kind, shape):
    """Forward on shapes the tile kernel takes, with NaN, infinities, signed zeros and exact ties
    planted in the data and in the thresholds; bit-exact against the oracle."""
    B, C, T, depth = shape
    x, thr, ord_, w = random_forest_inputs(7 + TILED_SHAPES.index(shape), kind, B, C, (), T, depth, (), quantise=True)
    rng = np.random.default_rng(3)
    flat = x.reshape(-1)
    for value in (np.nan, np.inf, -np.inf, 0.0, -0.0, 1e-42):
        flat[rng.choice(flat.size, max(4, flat.size // 50), replace=False)] = value
    tflat = thr.reshape(-1)
    for value in (np.nan, np.inf, -np.inf, 0.0, -0.0):
        tflat[rng.choice(tflat.size, max(1, tflat.size // 40), replace=False)] = value
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    f = cabi.Forest(kind, dx, dw)
    got = f.forward(dx, dthr, dord, dw).cpu().numpy()
    want = ho.forward(kind, x, thr, ord_, w)
    assert np.array_equal(got.view(np.uint32) & 0x7fffffff == 0, want.view(np.uint32) & 0x7fffffff == 0)
    assert np.array_equal(got, want, equal_nan=True)
    assert np.array_equal(f.leafmap(dx, dthr, dord).cpu().numpy(), ho.maps(kind, x, thr, ord_, w)[0])
    assert f.ordinal_flags() == 0


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", TILED_SHAPES, ids=[str(s) for s in TILED_SHAPES])
def test_tile_kernel_backward(cabi, kind, shape):
    """Default-mode backward on shapes the backward tile kernel takes (and on the wide ones it leaves to
    the any-shape kernel): within 1e-5 of the summed term magnitudes, with exact ties and zero margins."""
    B, C, T, depth = shape
    x, thr, ord_, w = random_forest_inputs(70 + TILED_SHAPES.index(shape), kind, B, C, (), T, depth, (), quantise=True)
    g = np.random.default_rng(4).standard_normal((B, T)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    f = cabi.Forest(kind, dx, dw)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    rx, rthr, rw = ho.backward(kind, x, thr, ord_, w, g)
    ax, athr, aw = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    assert grad_close(gx, rx, ax) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)
    assert f.ordinal_flags() == 0
    # with room for the evaluation records the tile path adds the x gradient in the reference's order in
    # both modes, and everything in that order in fixed-order mode: exact
    assert equal(gx, rx)
    fd = cabi.Forest(kind, dx, dw, deterministic=True)
    for got, ref in zip(fd.backward(dx, dthr, dord, dw, dg), (rx, rthr, rw)):
        assert equal(got, ref)
    # without that room: the scatter variant of the tile kernel (default mode), free summation order
    small = cabi.Forest(kind, dx, dw, backward_workspace=False)
    sx, sthr, sw = small.backward(dx, dthr, dord, dw, dg)
    assert grad_close(sx, rx, ax) and grad_close(sthr, rthr, athr) and grad_close(sw, rw, aw)
    # only some gradients requested
    only_w = f.backward(dx, dthr, dord, dw, dg, need=(False, False, True))
    assert only_w[0] is None and only_w[1] is None and grad_close(only_w[2], rw, aw)
    only_x = f.backward(dx, dthr, dord, dw, dg, need=(True, False, False))
    assert grad_close(only_x[0], rx, ax)


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("depth", [5, 8])
def test_large_batch_parameter_reduction_with_some_gradients(cabi, kind, depth):
    """From 65 536 samples on the default-mode parameter reduction keeps 16 lane-owned copies of a tree's bins and
    lets the two half-warps add different kinds of terms: a ragged batch of that size, with all gradients and with
    the threshold or the leaf-weight gradient alone."""
    B, C, T = 65536 + 100, 16, 8
    x, thr, ord_, w = random_forest_inputs(40 + depth, kind, B, C, (), T, depth, (), quantise=True)
    g = np.random.default_rng(8).standard_normal((B, T)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    rx, rthr, rw = ho.backward(kind, x, thr, ord_, w, g)
    ax, athr, aw = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    f = cabi.Forest(kind, dx, dw)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    assert equal(gx, rx) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)
    only_thr = f.backward(dx, dthr, dord, dw, dg, need=(False, True, False))
    assert only_thr[0] is None and only_thr[2] is None and grad_close(only_thr[1], rthr, athr)
    only_w = f.backward(dx, dthr, dord, dw, dg, need=(False, False, True))
    assert only_w[0] is None and only_w[1] is None and grad_close(only_w[2], rw, aw)
    assert f.ordinal_flags() == 0


MULTI_OUTPUT_SHAPES = [
    # B, C, T, depth, M: tabular input with several outputs per leaf (tile kernel, weights read from global memory)
    (4096, 256, 20, 10, 10),
    (700, 64, 50, 6, 3),
    (513, 300, 66, 5, 8),
    (300, 128, 130, 8, 2),
]


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", MULTI_OUTPUT_SHAPES, ids=[str(s) for s in MULTI_OUTPUT_SHAPES])
def test_tile_kernel_several_outputs_per_leaf(cabi, kind, shape):
    B, C, T, depth, M = shape
    x, thr, ord_, w = random_forest_inputs(90 + MULTI_OUTPUT_SHAPES.index(shape), kind, B, C, (), T, depth, (M,),
                                           quantise=True)
    x.reshape(-1)[::97] = np.nan
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    f = cabi.Forest(kind, dx, dw)
    got = f.forward(dx, dthr, dord, dw).cpu().numpy()
    assert got.shape == (B, T, M)
    assert np.array_equal(got, ho.forward(kind, x, thr, ord_, w), equal_nan=True)
    assert f.ordinal_flags() == 0


INNER_SHAPES = [
    # B, C, inner dims, T, depth: x [B, C, *inner] with one output per leaf, large enough for the tile kernel
    (8, 40, (64, 65), 20, 6),
    (3, 300, (1000,), 12, 5),      # more than 256 features: 16-bit feature indices
    (5, 16, (7, 11, 13), 9, 8),    # tiles straddle rows; positions not a multiple of 32
    (2, 128, (4099,), 33, 3),
    (700, 8, (3,), 70, 4),         # fewer positions than a warp
]


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", INNER_SHAPES, ids=[str(s) for s in INNER_SHAPES])
def test_tile_kernel_with_inner_positions(cabi, kind, shape):
    """Image-shaped inputs: a sample is a (row, position) pair; forward and maps bit-exact, ties and zeros included."""
    B, C, inner, T, depth = shape
    x, thr, ord_, w = random_forest_inputs(90 + INNER_SHAPES.index(shape), kind, B, C, inner, T, depth, (), quantise=True)
    x.reshape(-1)[:3] = [np.inf, -np.inf, np.nan]
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    f = cabi.Forest(kind, dx, dw)
    out = f.forward(dx, dthr, dord, dw)
    assert out.shape == (B, T) + tuple(inner)
    assert equal(out, ho.forward(kind, x, thr, ord_, w))
    leaf, margin, mord, reach = ho.maps(kind, x, thr, ord_, w)
    assert equal(f.leafmap(dx, dthr, dord), leaf)
    assert f.ordinal_flags() == 0


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", INNER_SHAPES, ids=[str(s) for s in INNER_SHAPES])
def test_tile_kernel_backward_with_inner_positions(cabi, kind, shape):
    """Record path on image-shaped inputs: default mode within tolerance (x gradient exact), fixed-order mode exact."""
    B, C, inner, T, depth = shape
    x, thr, ord_, w = random_forest_inputs(110 + INNER_SHAPES.index(shape), kind, B, C, inner, T, depth, (), quantise=True)
    g = np.random.default_rng(6).standard_normal((B, T) + tuple(inner)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    rx, rthr, rw = ho.backward(kind, x, thr, ord_, w, g)
    ax, athr, aw = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    f = cabi.Forest(kind, dx, dw)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    assert equal(gx, rx) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)
    fd = cabi.Forest(kind, dx, dw, deterministic=True)
    for got, ref in zip(fd.backward(dx, dthr, dord, dw, dg), (rx, rthr, rw)):
        assert equal(got, ref)
    small = cabi.Forest(kind, dx, dw, backward_workspace=False)  # scatter variant of the tile kernel
    sx, sthr, sw = small.backward(dx, dthr, dord, dw, dg)
    assert grad_close(sx, rx, ax) and grad_close(sthr, rthr, athr) and grad_close(sw, rw, aw)
    assert f.ordinal_flags() == 0


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("shape", MULTI_OUTPUT_SHAPES + [(257, 40, 130, 4, 33), (2100, 16, 20, 9, 64),
                                                        # from 4 Mi evaluations on: the tile kernel
                                                        (40000, 64, 110, 6, 3), (9000, 300, 500, 5, 33), (70001, 16, 64, 9, 64)],
                         ids=lambda s: str(s))
def test_tile_kernel_backward_several_outputs_per_leaf(cabi, kind, shape):
    """Default-mode backward with several outputs per leaf (tile kernel, work along the outputs shared by the warp)."""
    B, C, T, depth, M = shape
    x, thr, ord_, w = random_forest_inputs(130 + B % 97, kind, B, C, (), T, depth, (M,), quantise=True)
    g = np.random.default_rng(7).standard_normal((B, T, M)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    rx, rthr, rw = ho.backward(kind, x, thr, ord_, w, g)
    ax, athr, aw = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    f = cabi.Forest(kind, dx, dw)
    gx, gthr, gw = f.backward(dx, dthr, dord, dw, dg)
    assert grad_close(gx, rx, ax) and grad_close(gthr, rthr, athr) and grad_close(gw, rw, aw)
    only_w = f.backward(dx, dthr, dord, dw, dg, need=(False, False, True))
    assert only_w[0] is None and grad_close(only_w[2], rw, aw)
    only_x = f.backward(dx, dthr, dord, dw, dg, need=(True, False, False))
    assert grad_close(only_x[0], rx, ax) and only_x[2] is None
    fd = cabi.Forest(kind, dx, dw, deterministic=True)  # fixed-order mode: the ordered kernels, exact
    for got, ref in zip(fd.backward(dx, dthr, dord, dw, dg), (rx, rthr, rw)):
        assert equal(got, ref)
    assert f.ordinal_flags() == 0


SAVING_SHAPES = [
    # kind, B, C, T, depth: shapes the tile kernel takes with whole tree groups, and some it does not save for
    ("tree", 2048, 128, 64, 8, True),
    ("tree", 1999, 128, 48, 5, True),    # ragged last sample tile
    ("fern", 4096, 64, 32, 9, True),     # 16 + 16 bit vertex / leaf records
    ("tree", 700, 300, 128, 6, True),    # two-byte feature indices, smaller sample tiles
    ("tree", 2048, 128, 72, 8, False),   # short last tree group
    ("tree", 64, 16, 8, 4, False),       # too small for the tile kernel
]


@pytest.mark.parametrize("case", SAVING_SHAPES, ids=[str(c[:5]) for c in SAVING_SHAPES])
def test_backward_from_a_saved_forward(cabi, case):
    """forward(save) followed by backward(saved): the forward is the same bits, and the gradients computed from
    the kept traversal meet the same bars as those of the backward that walks the trees again (default mode within
    1e-5 of the summed magnitudes, fixed-order mode bit-exact).  Where the library does not save, the flags are
    ignored and the results are those of the plain calls."""
    kind, B, C, T, depth, saves = case
    x, thr, ord_, w = random_forest_inputs(SAVING_SHAPES.index(case) + 70, kind, B, C, (), T, depth, ())
    g = np.random.default_rng(9).standard_normal((B, T)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    want = ho.forward(kind, x, thr, ord_, w)
    ref = ho.backward(kind, x, thr, ord_, w, g)
    mags = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    for deterministic in (False, True):
        f = cabi.Forest(kind, dx, dw, deterministic=deterministic)
        assert f.saves_forward() == saves
        assert equal(f.forward(dx, dthr, dord, dw, save=True), want)
        got = f.backward(dx, dthr, dord, dw, dg, saved=True)
        for t, r, m in zip(got, ref, mags):
            assert equal(t, r) if deterministic else grad_close(t, r, m)
        # a subset of the gradients, from a fresh saved forward
        f.forward(dx, dthr, dord, dw, save=True)
        only_x = f.backward(dx, dthr, dord, dw, dg, need=(True, False, False), saved=True)
        assert only_x[1] is None and (equal(only_x[0], ref[0]) if deterministic else grad_close(only_x[0], ref[0], mags[0]))
        f.forward(dx, dthr, dord, dw, save=True)
        only_w = f.backward(dx, dthr, dord, dw, dg, need=(False, False, True), saved=True)
        assert only_w[0] is None and (equal(only_w[2], ref[2]) if deterministic else grad_close(only_w[2], ref[2], mags[2]))
        assert f.ordinal_flags() == 0
