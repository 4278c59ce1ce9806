"""Sparse-gradient operators and the hinge trie on a GPU.

Sparse operators: the COO gradients, densified, equal the dense operator's gradients exactly (the
values come from the same kernels), are coalesced, and hold exactly the elements the oracle says
receive a contribution.  Trie: forward bit-exact against the oracle and the reference's golden
vectors, gradients within rtol 1e-4 (atomic scatters)."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, random_forest_inputs
from oracle import hinge_oracle as ho

pytestmark = pytest.mark.gpu

FAMILIES = np.load(os.path.join(GOLDEN, "families.npz"))


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


def close(t, ref):
    return np.allclose(t.cpu().numpy(), ref, rtol=1e-4, atol=2e-5 * max(1.0, float(np.abs(ref).max())))


@pytest.mark.parametrize("kind", ["tree", "fern"])
def test_sparse_backward(kind):
    from hingetreefortorch_b200._ext import hingetree_cpp as ext
    x, thr, ord_, w = random_forest_inputs(31, kind, 12, 40, (2,), 6, 4, (3,))
    g = np.random.default_rng(0).standard_normal((12, 6, 2, 3)).astype(np.float32)
    dx, dthr, dord, dw, dg = dev(x, thr, ord_, w, g)
    sparse = getattr(ext, "sparse_%s_backward" % kind)(dx, True, dthr, True, dord, False, dw, True, dg)
    assert sparse[2] is None
    want = ho.backward(kind, x, thr, ord_, w, g)
    # which elements are touched: every (i,j,k) contributes to one x element, one threshold, M leaf weights
    ones = ho.backward(kind, x, thr, ord_, np.ones_like(w), np.ones_like(g))
    leaf, margin, mord, reach = ho.maps(kind, x, thr, ord_, w)
    for got, ref, name in zip((sparse[0], sparse[1], sparse[3]), want, ("x", "thr", "w")):
        assert got.is_sparse and got.is_coalesced() and got.shape == ref.shape
        assert close(got.to_dense(), ref), name
    touched_w = np.repeat((reach > 0)[..., None], 3, axis=-1)
    assert int(sparse[3]._nnz()) == int(touched_w.sum())
    dense_mask = torch.zeros(w.shape, dtype=torch.bool)
    idx = sparse[3].indices().cpu()
    dense_mask[idx[0], idx[1], idx[2]] = True
    assert np.array_equal(dense_mask.numpy(), touched_w)
    assert int(sparse[0]._nnz()) <= 12 * 6 * 2 and int(sparse[0]._nnz()) > 0


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
    assert close(gx, c["gx"]) and close(gthr, c["gthr"]) and close(gw, c["gw"])


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
    gx, gthr, gw = ho.trie_backward(x.detach().cpu().numpy(), m.thresholds.detach().cpu().numpy(), m.ordinals.cpu().numpy(),
                                    m.weights.detach().cpu().numpy(), np.ones(want.shape, np.float32))
    assert close(x.grad, gx) and close(m.thresholds.grad, gthr) and close(m.weights.grad, gw)
