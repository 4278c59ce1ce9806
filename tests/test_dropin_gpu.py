"""The reference-facing surface on a GPU: the `hingetree_cpp` operators, the autograd
Functions and the nn.Modules, checked against the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import grad_close, random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from hingetreefortorch_b200._ext import hingetree_cpp
    return hingetree_cpp


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_operators_match_oracle(ext, kind):
    x, thr, ord_, w = random_forest_inputs(21, kind, 40, 12, (3,), 10, 4, (2,))
    g = np.random.default_rng(0).standard_normal((40, 10, 3, 2)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    out = getattr(ext, kind + "_forward")(dx, dthr, dord, dw)
    assert out.shape == (40, 10, 3, 2) and np.array_equal(out.cpu().numpy(), ho.forward(kind, x, thr, ord_, w))
    leaf, margin, mord, reach = ho.maps(kind, x, thr, ord_, w)
    got_leaf = getattr(ext, kind + "_leafmap")(dx, dthr, dord, dw)
    assert got_leaf.dtype == torch.int64 and np.array_equal(got_leaf.cpu().numpy(), leaf)
    got_margin, got_mord = getattr(ext, kind + "_marginmap")(dx, dthr, dord, dw)
    assert np.array_equal(got_margin.cpu().numpy(), margin) and np.array_equal(got_mord.cpu().numpy(), mord)
    got_reach = getattr(ext, kind + "_reachability")(dx, dthr, dord, dw)
    assert got_reach.dtype == torch.int64 and np.array_equal(got_reach.cpu().numpy(), reach)
    want = ho.backward(kind, x, thr, ord_, w, g)
    grads = getattr(ext, kind + "_backward_deterministic")(dx, True, dthr, True, dord, False, dw, True, dg)
    assert grads[2] is None
    for got, ref in zip((grads[0], grads[1], grads[3]), want):
        assert np.array_equal(got.cpu().numpy(), ref)
    grads = getattr(ext, kind + "_backward")(dx, True, dthr, False, dord, False, dw, True, dg)
    assert grads[1] is None and grads[2] is None
    mags = ho.backward_magnitudes(kind, x, thr, ord_, w, g)
    assert grad_close(grads[0], want[0], mags[0]) and grad_close(grads[3], want[2], mags[2])
    assert getattr(ext, kind + "_backward")(dx, False, dthr, False, dord, False, dw, False, dg) == [None] * 4


def test_module_training_step_keeps_the_forward_traversal(ext):
    """A module large enough for the tile kernel: the autograd Function keeps the forward's traversal and the
    backward uses it (ext.tree_forward_saving returns a non-empty scratch); results match the oracle at the
    usual bars, in default and in deterministic mode, and equal those with keeping switched off."""
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(3)
    m = R.RandomHingeForest(128, 64, 6, extra_outputs=1).cuda()
    x = torch.randn(1024, 128, device="cuda", requires_grad=True)
    w2 = m.weights.detach().reshape(64, 64)
    assert ext.tree_forward_saving(x.detach(), m.thresholds.detach(), m.ordinals, w2)[1].numel() > 0
    results = {}
    for keep in (True, False):
        ext.set_save_forward(keep)
        try:
            for p in (x, m.thresholds, m.weights):
                p.grad = None
            y = m(x)
            (y * y).sum().backward()
            results[keep] = [t.detach().clone() for t in (y, x.grad, m.thresholds.grad, m.weights.grad)]
        finally:
            ext.set_save_forward(True)
    xn, thr, ord_, w = x.detach().cpu().numpy(), m.thresholds.detach().cpu().numpy(), m.ordinals.cpu().numpy(), m.weights.detach().cpu().numpy()
    want = ho.forward("tree", xn, thr, ord_, w)
    g = 2 * want
    ref = ho.backward("tree", xn, thr, ord_, w, g)
    mags = ho.backward_magnitudes("tree", xn, thr, ord_, w, g)
    for keep in (True, False):
        assert np.array_equal(results[keep][0].cpu().numpy(), want)
        for t, r, mg in zip(results[keep][1:], ref, mags):
            assert grad_close(t, r, mg)
    assert torch.equal(results[True][1], results[False][1])  # the x gradient is added in tree order either way
    prev = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        for p in (x, m.thresholds, m.weights):
            p.grad = None
        y = m(x)
        (y * y).sum().backward()
    finally:
        torch.use_deterministic_algorithms(prev)
    for t, r in zip((x.grad, m.thresholds.grad, m.weights.grad), ref):
        assert np.array_equal(t.cpu().numpy(), r)


def test_error_contract_on_device(ext):
    x, thr, ord_, w = random_forest_inputs(22, "tree", 8, 5, (), 3, 3, ())
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    bad = dord.clone()
    bad[0, 0] = 5
    with pytest.raises(RuntimeError, match="ordinal"):
        ext.tree_forward(dx, dthr, bad, dw)
    with pytest.raises(RuntimeError, match="ordinal"):
        ext.tree_backward(dx, True, dthr, True, bad, False, dw, True, torch.ones(8, 3, device="cuda"))
    with pytest.raises(ValueError, match="same device"):
        ext.tree_forward(dx, dthr.cpu(), dord, dw)
    with pytest.raises(RuntimeError, match="tree depth"):
        ext.tree_forward(dx, dthr[:, :6].contiguous(), dord[:, :6].contiguous(), dw)
    with pytest.raises(ValueError, match="outDataGrad.shape"):
        ext.tree_backward(dx, True, dthr, True, dord, False, dw, True, torch.ones(8, 4, device="cuda"))
    with pytest.raises(ValueError):  # mixed real types
        ext.tree_forward(dx.double(), dthr, dord, dw)
    with pytest.raises(ValueError):  # half precision is taken by no operator
        ext.tree_forward(dx.half(), dthr.half(), dord, dw.half())
    # a valid ordinals tensor that is later corrupted in place is re-validated (version changed)
    ext.tree_forward(dx, dthr, dord, dw)
    dord[1, 1] = -3
    with pytest.raises(RuntimeError, match="ordinal"):
        ext.tree_forward(dx, dthr, dord, dw)


@pytest.mark.parametrize("module_name,kind", [("RandomHingeForest", "tree"), ("RandomHingeFern", "fern")])
def test_modules_forward_backward(module_name, kind):
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(0)
    m = getattr(R, module_name)(20, 16, 5, extra_outputs=3).cuda()
    x = torch.randn(64, 20, device="cuda", requires_grad=True)
    y = m(x)
    assert y.shape == (64, 16, 3)
    y.backward(torch.ones_like(y))
    xn, thr, ord_, w = x.detach().cpu().numpy(), m.thresholds.detach().cpu().numpy(), m.ordinals.cpu().numpy(), m.weights.detach().cpu().numpy()
    assert np.array_equal(y.detach().cpu().numpy(), ho.forward(kind, xn, thr, ord_, w))
    gx, gthr, gw = ho.backward(kind, xn, thr, ord_, w, np.ones(y.shape, np.float32))
    ax, athr, aw = ho.backward_magnitudes(kind, xn, thr, ord_, w, np.ones(y.shape, np.float32))
    assert grad_close(x.grad, gx, ax) and grad_close(m.thresholds.grad, gthr, athr) and grad_close(m.weights.grad, gw, aw)
    assert m.ordinals.grad is None
    # deterministic mode selects the fixed-order backward: bit-exact against the oracle
    prev = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        for p in (x, m.thresholds, m.weights):
            p.grad = None
        m(x).backward(torch.ones_like(y))
    finally:
        torch.use_deterministic_algorithms(prev)
    assert np.array_equal(x.grad.cpu().numpy(), gx)
    assert np.array_equal(m.thresholds.grad.cpu().numpy(), gthr)
    assert np.array_equal(m.weights.grad.cpu().numpy(), gw)
    # analysis helpers
    leaf = m.leafmap(x.detach())
    assert leaf.shape == (64, 16) and m.reachability(x.detach()).sum() == 64 * 16
    assert m.pathmap(x.detach()).shape == (64, 16, 5)


def test_kernels_run_on_the_current_stream(ext):
    x, thr, ord_, w = random_forest_inputs(23, "tree", 512, 64, (), 32, 6, ())
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    ext.tree_forward(dx, dthr, dord, dw)  # validates the ordinals once
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        out = ext.tree_forward(dx, dthr, dord, dw)
    side.synchronize()
    assert np.array_equal(out.cpu().numpy(), ho.forward("tree", x, thr, ord_, w))


def test_training_step_is_cuda_graph_capturable():
    """Once an ordinals tensor has been validated no operator synchronises or reads back, so a whole
    forward + backward of a module can be captured in a CUDA graph and replayed on new data."""
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(3)
    m = R.RandomHingeForest(40, 12, 5, extra_outputs=2).cuda()
    x = torch.rand(64, 40, device="cuda", requires_grad=True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # validates the ordinals, warms the allocator
            m(x).sum().backward()
    torch.cuda.current_stream().wait_stream(side)
    m.zero_grad(set_to_none=True)
    x.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = m(x)
        y.sum().backward()
    with torch.no_grad():
        x.copy_(torch.rand(64, 40, device="cuda"))  # new data in the captured input
    graph.replay()
    torch.cuda.synchronize()
    got_y, got_gx, got_gw = y.clone(), x.grad.clone(), m.weights.grad.clone()
    m.zero_grad(set_to_none=True)
    x.grad = None
    want = m(x)
    want.sum().backward()
    assert torch.equal(got_y, want)
    assert torch.allclose(got_gx, x.grad, rtol=1e-5, atol=1e-6) and torch.allclose(got_gw, m.weights.grad, rtol=1e-5, atol=1e-6)


def test_backward_scratch_limit_switches_to_scatters(ext):
    """With the per-evaluation records ruled out the default-mode backward still matches within tolerance."""
    rng = np.random.default_rng(8)
    B, C, T, depth = 1200, 64, 40, 6
    x = rng.standard_normal((B, C)).astype(np.float32)
    thr = rng.uniform(-3, 3, (T, 63)).astype(np.float32)
    ord_ = rng.integers(0, C, (T, 63)).astype(np.int64)
    w = rng.standard_normal((T, 64)).astype(np.float32)
    g = rng.standard_normal((B, T)).astype(np.float32)
    dx, dthr, dord, dw, dg = [torch.from_numpy(a).cuda() for a in (x, thr, ord_, w, g)]
    with_records = ext.tree_backward(dx, True, dthr, True, dord, False, dw, True, dg)
    ext.set_backward_scratch_limit(0)
    try:
        scattered = ext.tree_backward(dx, True, dthr, True, dord, False, dw, True, dg)
    finally:
        ext.set_backward_scratch_limit(2 ** 62)
    want = ho.backward("tree", x, thr, ord_, w, g)
    mags = ho.backward_magnitudes("tree", x, thr, ord_, w, g)
    for got in (with_records, scattered):  # both paths against the oracle at the stated bar
        for t, ref, mag in zip((got[0], got[1], got[3]), want, mags):
            assert grad_close(t, ref, mag)
    with pytest.raises(ValueError):
        ext.set_backward_scratch_limit(-1)


def test_speedtest_sweeps_like_the_reference(ext, capfd):
    """The reference's own benchmark operator: trees 1..512 by powers of two, depth 1..12, rows = trees, depth,
    forward ms, backward ms (hingetree.cpp:1361-1438)."""
    x = torch.rand(100, 1000, device="cuda")
    timings = ext.tree_speedtest(x, False)
    assert timings.shape == (4, 120) and timings.device.type == "cpu"
    assert timings[0].tolist() == [float(2 ** s) for s in range(10) for _ in range(12)]
    assert timings[1].tolist() == [float(d) for _ in range(10) for d in range(1, 13)]
    assert bool((timings[2:] > 0).all()) and float(timings[2:].max()) < 50.0
    assert "hingetree_forward: numBatches = 100" in capfd.readouterr().out


def test_a_wait_that_runs_out_reaches_the_caller(ext):
    """The error path of the tile kernels without a lost copy: the library's self-test kernel waits a few tries on
    a barrier nothing arrives on, sets HT_FLAG_PIPELINE_TIMEOUT and returns; the C ABI shows the flag in the
    caller's status word, the extension raises RuntimeError at its next status read and clears the word, and the
    device keeps working."""
    from hingetreefortorch_b200 import _cabi
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    _cabi.selftest_bounded_wait(status)
    assert int(status.item()) & _cabi.HT_FLAG_PIPELINE_TIMEOUT
    assert ext.pipeline_status() == 0
    ext.selftest_bounded_wait()
    with pytest.raises(RuntimeError, match="bounded wait"):
        ext.pipeline_status()
    assert ext.pipeline_status() == 0
    x, thr, ord_, w = random_forest_inputs(3, "tree", 16, 8, (), 4, 3, ())
    dx, dthr, dord, dw = dev(x, thr, ord_, w)
    assert np.array_equal(ext.tree_forward(dx, dthr, dord, dw).cpu().numpy(), ho.forward("tree", x, thr, ord_, w))
