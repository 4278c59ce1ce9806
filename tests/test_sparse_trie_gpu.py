"""Sparse-gradient operators and the hinge trie on a GPU.

Sparse operators: the COO gradients, densified, equal the dense operator's gradients exactly (the
values come from the same kernels), are coalesced, and hold exactly the elements the oracle says
receive a contribution.  Trie: forward bit-exact against the oracle and the reference's golden
vectors, gradients (summation order is free) within 1e-5 of the summed term magnitudes.  The sparse
fused-linear operator is checked value by value against the oracle as well."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, grad_close, random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu

FAMILIES = np.load(os.path.join(GOLDEN, "families.npz"))


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_sparse_backward(kind):
    from hingetreefortorch_b200._ext import hingetree_cpp as ext
    x, thr, ord_, w = random_forest_inputs(31, kind, 12, 40, (2,), 6, 4, (3,))
    g = np.random.default_rng(0).standard_normal((12, 6, 2, 3)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    sparse = getattr(ext, "sparse_%s_backward" % kind)(dx, True, dthr, True, dord, False, dw, True, dg)
    assert sparse[2] is None
    want = ho.backward(kind, x, thr, ord_, w, g)
    scale = ho.magnitudes(ho.backward, kind, x, thr, ord_, w, g)
    # which elements are touched: every (i,j,k) contributes to one x element, one threshold, M leaf weights
    ones = ho.backward(kind, x, thr, ord_, np.ones_like(w), np.ones_like(g))
    leaf, margin, mord, reach = ho.maps(kind, x, thr, ord_, w)
    for got, ref, mag, name in zip((sparse[0], sparse[1], sparse[3]), want, scale, ("x", "thr", "w")):
        assert got.is_sparse and got.is_coalesced() and got.shape == ref.shape
        assert grad_close(got.to_dense(), ref, mag), name
    touched_w = np.repeat((reach > 0)[..., None], 3, axis=-1)
    assert int(sparse[3]._nnz()) == int(touched_w.sum())
    dense_mask = torch.zeros(w.shape, dtype=torch.bool)
    idx = sparse[3].indices().cpu()
    dense_mask[idx[0], idx[1], idx[2]] = True
    assert np.array_equal(dense_mask.numpy(), touched_w)
    assert int(sparse[0]._nnz()) <= 12 * 6 * 2 and int(sparse[0]._nnz()) > 0


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_sparse_fused_linear_backward_values(kind):
    """sparse_*_fused_linear_backward: x / threshold / leaf-weight gradients come back as coalesced COO tensors
    whose dense form equals the oracle's fused-linear backward, with exactly the touched elements stored;
    the linear weight and bias gradients stay dense."""
    from hingetreefortorch_b200._ext import hingetree_cpp as ext
    x, thr, ord_, w = random_forest_inputs(37, kind, 10, 30, (3,), 7, 4, (2,))
    rng = np.random.default_rng(3)
    O = 5
    lin = rng.standard_normal((O, 7)).astype(np.float32)
    bias = rng.standard_normal(O).astype(np.float32)
    g = rng.standard_normal((10, O, 3, 2)).astype(np.float32)
    dx, dthr, dord, dw, dlin, dbias, dg = dev(x, thr, ord_, w, lin, bias, g)
    got = getattr(ext, "sparse_%s_fused_linear_backward" % kind)(dx, True, dthr, True, dord, False, dw, True, dlin, True,
                                                                  dbias, True, dg)
    assert len(got) == 6 and got[2] is None
    rx, rthr, rw, rlin, rbias = ho.linear_backward(kind, x, thr, ord_, w, lin, g)
    ax, athr, aw, alin, abias = ho.magnitudes(ho.linear_backward, kind, x, thr, ord_, w, lin, g)
    for t, ref, mag, name in ((got[0], rx, ax, "x"), (got[1], rthr, athr, "thr"), (got[3], rw, aw, "w")):
        assert t.is_sparse and t.is_coalesced() and t.shape == ref.shape, name
        assert grad_close(t.to_dense(), ref, mag), name
    assert not got[4].is_sparse and grad_close(got[4], rlin, alin)
    assert not got[5].is_sparse and grad_close(got[5], rbias, abias)
    # stored pattern of the leaf-weight gradient: every output of every leaf some position reaches
    reach = ho.maps(kind, x, thr, ord_, w)[3]
    touched_w = np.repeat((reach > 0)[..., None], 2, axis=-1)
    mask = torch.zeros(w.shape, dtype=torch.bool)
    idx = got[3].indices().cpu()
    mask[idx[0], idx[1], idx[2]] = True
    assert np.array_equal(mask.numpy(), touched_w)
    # thresholds: exactly the deciding vertices
    leaf, margin, mord, _ = ho.maps(kind, x, thr, ord_, w)
    assert 0 < int(got[1]._nnz()) <= thr.size and int(got[0]._nnz()) <= 10 * 7 * 3


def test_sparse_modules_train_step():
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(4)
    m = R.SparseRandomHingeForest(30, 8, 4).cuda()
    x = torch.randn(16, 30, device="cuda", requires_grad=True)
    m(x).sum().backward()
    assert not x.grad.is_sparse and m.thresholds.grad.is_sparse and m.weights.grad.is_sparse
    dense = R.RandomHingeForest(30, 8, 4).cuda()
    dense.load_state_dict(m.state_dict())
    x2 = x.detach().clone().requires_grad_(True)
    dense(x2).sum().backward()
    assert torch.allclose(x.grad, x2.grad, rtol=1e-5, atol=1e-6)
    assert torch.allclose(m.weights.grad.to_dense(), dense.weights.grad, rtol=1e-5, atol=1e-6)
    fl = R.SparseRandomHingeFernFusedLinear(30, 8, 3, 4).cuda()
    x3 = x.detach().clone().requires_grad_(True)
    fl(x3).sum().backward()
    assert fl.weights.grad.is_sparse and not fl.linear_weights.grad.is_sparse and not x3.grad.is_sparse


@pytest.mark.parametrize("idx", range(int(FAMILIES["trie_count"])))
def test_trie_golden(idx):
    from hingetreefortorch_b200._ext import hingetree_cpp as ext
    n = len("trie%02d_" % idx)
    c = {k[n:]: FAMILIES[k] for k in FAMILIES.files if k.startswith("trie%02d_" % idx)}
    d = {k: dev(v)[0] for k, v in c.items()}
    out = ext.trie_forward(d["x"], d["thr"], d["ord"], d["w"])
    assert np.array_equal(out.cpu().numpy(), c["out"])
    gx, gthr, _, gw = ext.trie_backward(d["x"], True, d["thr"], True, d["ord"], False, d["w"], True, d["g"])
    ax, athr, aw = ho.magnitudes(ho.trie_backward, c["x"], c["thr"], c["ord"], c["w"], c["g"])
    assert grad_close(gx, c["gx"], ax) and grad_close(gthr, c["gthr"], athr) and grad_close(gw, c["gw"], aw)


def test_trie_module_and_larger_shape():
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(6)
    m = R.RandomHingeTrie(20, 10, 6, extra_outputs=2).cuda()
    x = torch.randn(50, 20, device="cuda", requires_grad=True)
    y = m(x)
    assert y.shape == (50, 10, 2)
    y.sum().backward()
    want = ho.trie_forward(x.detach().cpu().numpy(), m.thresholds.detach().cpu().numpy(), m.ordinals.cpu().numpy(),
                           m.weights.detach().cpu().numpy())
    assert np.array_equal(y.detach().cpu().numpy(), want)
    args = (x.detach().cpu().numpy(), m.thresholds.detach().cpu().numpy(), m.ordinals.cpu().numpy(),
            m.weights.detach().cpu().numpy(), np.ones(want.shape, np.float32))
    gx, gthr, gw = ho.trie_backward(*args)
    ax, athr, aw = ho.magnitudes(ho.trie_backward, *args)
    assert grad_close(x.grad, gx, ax) and grad_close(m.thresholds.grad, gthr, athr) and grad_close(m.weights.grad, gw, aw)
