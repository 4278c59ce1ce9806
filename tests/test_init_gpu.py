"""Threshold initialisation and hygiene on the device (`ht_init_medians_*`, `ht_thresholds_*`): the operators the
reference runs on CPU tensors only, given CUDA tensors.  Checked against the golden vectors of the unmodified
reference (tests/golden/init.npz) and against this library's host operators, bit for bit."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from hingetreefortorch_b200._ext import hingetree_cpp
    return hingetree_cpp


def test_median_initialisation_on_the_device_matches_the_reference(ext):
    golden = np.load(os.path.join(GOLDEN, "init.npz"))
    for idx in range(int(golden["count"])):
        p = "init%02d_" % idx
        family = str(golden[p + "family"])
        x, thr, ord_, w = [torch.from_numpy(golden[p + k].copy()).cuda() for k in ("x", "thr", "ord", "w")]
        ok = getattr(ext, family + "_init_medians")(x, thr, ord_, w)
        assert ok == bool(golden[p + "ok"])
        assert np.array_equal(thr.cpu().numpy(), golden[p + "after"]), (idx, family)


@pytest.mark.parametrize("family", ["tree", "fern", "trie"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape", [(500, 20, ()), (37, 6, (5, 3)), (3, 4, ()), (20000, 64, ())])
def test_median_initialisation_device_equals_host(ext, family, dtype, shape):
    """Few samples (vertices nobody reaches keep their threshold), many samples, inner positions, ties (values
    rounded to halves), both precisions; the C ABI directly and the extension."""
    from hingetreefortorch_b200 import _cabi
    B, C, inner = shape
    gen = torch.Generator().manual_seed(B + C)
    depth, T = 5, 9
    N = depth if family == "fern" else 2 ** depth - 1
    x = torch.randn((B, C) + inner, generator=gen, dtype=dtype)
    x = torch.where(torch.rand(x.shape, generator=gen) < 0.3, torch.round(x * 2) / 2 + 0.25, x)  # ties
    thr = torch.rand((T, N), generator=gen, dtype=dtype) * 6 - 3
    ord_ = torch.randint(0, C, (T, N), generator=gen)
    w = torch.zeros((T, 2 ** depth - 1 if family == "trie" else 2 ** depth, 2), dtype=dtype)
    host = thr.clone()
    assert getattr(ext, family + "_init_medians")(x, host, ord_, w) is True
    device = thr.clone().cuda()
    assert getattr(ext, family + "_init_medians")(x.cuda(), device, ord_.cuda(), w.cuda()) is True
    assert torch.equal(device.cpu(), host)
    direct = thr.clone().cuda()
    _cabi.init_medians("fern" if family == "fern" else "tree", x.cuda(), direct, ord_.cuda())
    assert torch.equal(direct.cpu(), host)


def test_median_initialisation_screens_on_the_device(ext):
    x = torch.randn(9, 4).cuda()
    thr, ord_, w = torch.zeros(2, 7).cuda(), torch.randint(0, 4, (2, 7)).cuda(), torch.zeros(2, 8).cuda()
    before = thr.clone()
    bad = ord_.clone()
    bad[1, 3] = 4  # feature index beyond the data: False, nothing written
    assert ext.tree_init_medians(x, thr, bad, w) is False and torch.equal(thr, before)
    with pytest.raises(ValueError):
        ext.tree_init_medians(x, thr.cpu(), ord_, w)  # mixed devices
    from hingetreefortorch_b200 import RandomHingeForest as R
    forest = R.RandomHingeForest(4, 3, 3).cuda()
    assert forest.init_medians(x) is True
    root = forest.ordinals[:, 0]
    medians = torch.stack([x[:, c].sort(descending=True).values[9 // 2] for c in root.tolist()])
    assert torch.equal(forest.thresholds.data[:, 0], medians)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_threshold_check_and_fix_device_equal_host(ext, dtype):
    """Few features and deep trees: most vertices share a feature with an ancestor, many thresholds are out of
    their reachable interval."""
    gen = torch.Generator().manual_seed(11)
    T, depth = 300, 6
    N = 2 ** depth - 1
    thr = (torch.rand((T, N), generator=gen, dtype=dtype) * 6 - 3)
    ord_ = torch.randint(0, 3, (T, N), generator=gen)
    ord_[:40] = torch.arange(N) % 64  # trees without repeated features on any path: consistent as they are
    w = torch.zeros((T, 2 ** depth), dtype=dtype)
    host, device = thr.clone(), thr.clone().cuda()
    assert ext.tree_check_thresholds(device, ord_.cuda(), w.cuda()) == ext.tree_check_thresholds(host, ord_, w)
    changed_host = ext.tree_fix_thresholds(host, ord_, w)
    changed_device = ext.tree_fix_thresholds(device, ord_.cuda(), w.cuda())
    assert changed_device == changed_host and any(changed_host) and not all(changed_host)
    assert torch.equal(device.cpu(), host)
    assert all(ext.tree_check_thresholds(device, ord_.cuda(), w.cuda()))
    assert ext.fern_check_thresholds(device[:, :depth].contiguous(), ord_[:, :depth].contiguous().cuda(), w.cuda()) == [True] * T
