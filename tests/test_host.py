"""Host-side logic of the drop-in that needs no GPU: the torch extension loads, exposes the
reference's operator names, screens arguments with the reference's exception types, and the
threshold-hygiene utilities reproduce the reference on the golden vectors."""
import numpy as np
import pytest
import torch

from hingetreefortorch_b200._ext import hingetree_cpp
from hingetreefortorch_b200 import HingeTree as F, RandomHingeForest as R

REFERENCE_OPERATORS = """
tree_forward tree_backward tree_backward_deterministic sparse_tree_backward tree_check_thresholds tree_fix_thresholds
tree_reachability tree_leafmap tree_marginmap tree_speedtest tree_init_medians tree_init_greedy
fern_forward fern_backward fern_backward_deterministic sparse_fern_backward fern_check_thresholds fern_fix_thresholds
fern_reachability fern_leafmap fern_marginmap fern_speedtest fern_init_medians
tree_conv1d_forward tree_conv2d_forward tree_conv3d_forward tree_conv1d_backward tree_conv2d_backward tree_conv3d_backward
fern_conv1d_forward fern_conv2d_forward fern_conv3d_forward fern_conv1d_backward fern_conv2d_backward fern_conv3d_backward
trie_forward trie_backward trie_init_medians
tree_fused_linear_forward tree_fused_linear_backward sparse_tree_fused_linear_backward
fern_fused_linear_forward fern_fused_linear_backward sparse_fern_fused_linear_backward
tree_fusion_forward tree_fusion_backward fern_fusion_forward fern_fusion_backward
tree_fusion_fused_linear_forward tree_fusion_fused_linear_backward
fern_fusion_fused_linear_forward fern_fusion_fused_linear_backward contract expand
""".split()


def test_extension_exposes_the_reference_operator_names():
    assert len(REFERENCE_OPERATORS) == 54
    for name in REFERENCE_OPERATORS:
        assert callable(getattr(hingetree_cpp, name)), name


def test_threshold_hygiene_matches_reference(golden_forest):
    g = golden_forest
    thr = torch.from_numpy(g["hygiene_thr_before"].copy())
    ord_ = torch.from_numpy(g["hygiene_ord"])
    w = torch.zeros(thr.shape[0], thr.shape[1] + 1)
    assert hingetree_cpp.tree_check_thresholds(thr, ord_, w) == g["hygiene_check_before"].tolist()
    assert hingetree_cpp.tree_fix_thresholds(thr, ord_, w) == g["hygiene_changed"].tolist()
    assert np.array_equal(thr.numpy(), g["hygiene_thr_after"])
    assert hingetree_cpp.tree_check_thresholds(thr, ord_, w) == g["hygiene_check_after"].tolist()
    assert all(g["hygiene_check_after"].tolist())
    # ferns: nothing to check, nothing to fix
    thr_f, ord_f, w_f = torch.randn(3, 4), torch.randint(0, 5, (3, 4)), torch.randn(3, 16)
    assert hingetree_cpp.fern_check_thresholds(thr_f, ord_f, w_f) == [True] * 3
    assert hingetree_cpp.fern_fix_thresholds(thr_f, ord_f, w_f) == [False] * 3


def test_argument_screening_uses_the_reference_exception_types():
    x, thr, ord_, w = torch.randn(4, 5), torch.randn(3, 7), torch.randint(0, 5, (3, 7)), torch.randn(3, 8)
    with pytest.raises(ValueError):  # dtype mismatch
        hingetree_cpp.tree_forward(x.double(), thr, ord_, w)
    with pytest.raises(ValueError):  # ordinals must be int64
        hingetree_cpp.tree_forward(x, thr, ord_.int(), w)
    with pytest.raises(ValueError):  # not contiguous
        hingetree_cpp.tree_forward(x.t().contiguous().t(), thr, ord_, w)
    with pytest.raises(RuntimeError, match="CUDA devices only"):  # no CPU evaluation path
        hingetree_cpp.tree_forward(x, thr, ord_, w)
    with pytest.raises(RuntimeError, match="inOrdinals never has a gradient"):
        hingetree_cpp.tree_backward(x, True, thr, True, ord_, True, w, True, torch.randn(4, 3))
    with pytest.raises(ValueError):
        hingetree_cpp.tree_check_thresholds(thr, ord_.int(), w)
    with pytest.raises(RuntimeError):  # 7 thresholds do not fit 16 leaves
        hingetree_cpp.tree_check_thresholds(thr, ord_, torch.randn(3, 16))


def test_modules_construct_like_the_reference():
    torch.manual_seed(3)
    m = R.RandomHingeForest(10, 4, 3, extra_outputs=1)
    assert m.weights.shape == (4, 8, 1) and m.thresholds.shape == (4, 7) and m.ordinals.dtype == torch.long
    assert not m.ordinals.requires_grad and all(m.check_thresholds())
    assert list(m.state_dict().keys()) == ["weights", "thresholds", "ordinals"]
    assert R.RandomHingeFern(10, 4, 5, extra_outputs=[2, 3]).weights.shape == (4, 32, 2, 3)
    seq = R.RandomHingeForest(12700, 100, 7, init_type="sequential")
    assert torch.equal(seq.ordinals, torch.arange(12700).view(100, 127))
    fl = R.RandomHingeForestFusedLinear(10, 6, 3, 4, bias=False)
    assert fl.linear_weights.shape == (3, 6) and not fl.linear_bias.requires_grad
    fu = R.RandomHingeFernFusion(5, 3, 6, 4)
    assert fu.ordinals.shape == (6, 4) and int(fu.ordinals.max()) < 8
    conv = R.HingeTreeConv2d(3, 4, 2, 3, padding=1, extra_outputs=5)
    assert conv.thresholds.shape == (4, 3, 3) and conv.weights.shape == (4, 3, 4, 5) and int(conv.ordinals.max()) < 9
    with pytest.raises(RuntimeError):
        R.RandomHingeForest(10, 4, 3, init_type="nope")
    # checkpoints that store the ordinals as float32 load and are cast back to long
    state = {k: v.clone() for k, v in m.state_dict().items()}
    state["ordinals"] = state["ordinals"].float()
    m2 = R.RandomHingeForest(10, 4, 3, extra_outputs=1)
    m2.ordinals = torch.nn.Parameter(m2.ordinals.float(), requires_grad=False)
    m2.load_state_dict(state)
    assert m2.ordinals.dtype == torch.long and torch.equal(m2.ordinals, m.ordinals)


def test_function_layer_names():
    for name in ["HingeTree", "HingeFern", "SparseHingeTree", "SparseHingeFern", "HingeTreeFusedLinear",
                 "HingeFernFusedLinear", "SparseHingeTreeFusedLinear", "SparseHingeFernFusedLinear", "HingeTreeFusion",
                 "HingeFernFusion", "HingeTreeFusionFusedLinear", "HingeFernFusionFusedLinear", "HingeTreeConv1d",
                 "HingeTreeConv2d", "HingeTreeConv3d", "HingeFernConv1d", "HingeFernConv2d", "HingeFernConv3d",
                 "HingeTrie", "contract", "expand", "Contract", "Expand"]:
        assert hasattr(F, name), name
    assert issubclass(F.SparseHingeTree, F.HingeTree) and issubclass(F.HingeTreeFusedLinear, F.HingeTree)


def test_median_initialisation_matches_reference():
    """init_medians (CPU tensors, in place) against thresholds produced by the unmodified reference, bit for bit."""
    import os
    golden = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "init.npz"))
    for idx in range(int(golden["count"])):
        p = "init%02d_" % idx
        family = str(golden[p + "family"])
        x, thr, ord_, w = [torch.from_numpy(golden[p + k].copy()) for k in ("x", "thr", "ord", "w")]
        ok = getattr(hingetree_cpp, family + "_init_medians")(x, thr, ord_, w)
        assert ok == bool(golden[p + "ok"])
        assert np.array_equal(thr.numpy(), golden[p + "after"]), (idx, family)


def test_median_initialisation_screens_like_the_reference():
    x = torch.randn(9, 4)
    thr, ord_, w = torch.zeros(2, 7), torch.randint(0, 4, (2, 7)), torch.zeros(2, 8)
    before = thr.clone()
    bad = ord_.clone()
    bad[1, 3] = 4                                    # feature index beyond the data: False, nothing written
    assert hingetree_cpp.tree_init_medians(x, thr, bad, w) is False and torch.equal(thr, before)
    assert hingetree_cpp.tree_init_medians(x, torch.zeros(2, 6), ord_[:, :6].contiguous(), w) is False
    with pytest.raises(ValueError):
        hingetree_cpp.tree_init_medians(x.double(), thr, ord_, w)
    with pytest.raises(ValueError):
        hingetree_cpp.fern_init_medians(x, thr, ord_.int(), w)
    forest = R.RandomHingeForest(4, 3, 3)
    assert forest.init_medians(x) is True
    root = forest.ordinals[:, 0]
    medians = torch.stack([x[:, c].sort(descending=True).values[9 // 2] for c in root.tolist()])
    assert torch.equal(forest.thresholds.data[:, 0], medians)


def test_greedy_initialisation_grows_trees_that_separate_the_classes():
    """tree_init_greedy draws at random (as the reference's does), so the check is on what any correct run
    must give: valid trees, reproducible after seed_init, unsplittable vertices closed off, purer leaves."""
    gen = torch.Generator().manual_seed(0)
    B, C, T = 400, 9, 6
    x = torch.randn(B, C, generator=gen)
    y = (x[:, 3] > 0.2).long() + 2 * (x[:, 5] < -0.1).long()          # 4 classes, decided by features 3 and 5
    thr, ord_, w = torch.zeros(T, 7), torch.randint(0, C, (T, 7), generator=gen), torch.zeros(T, 8)
    hingetree_cpp.seed_init(7)
    assert hingetree_cpp.tree_init_greedy(x, y, thr, ord_, w) is True
    assert int(ord_.min()) >= 0 and int(ord_.max()) < C and not torch.isnan(thr).any()
    thr2, ord2 = torch.zeros(T, 7), torch.randint(0, C, (T, 7), generator=gen)
    hingetree_cpp.seed_init(7)
    assert hingetree_cpp.tree_init_greedy(x, y, thr2, ord2, w) and torch.equal(thr, thr2) and torch.equal(ord_, ord2)

    def leaves(tree):
        v = torch.zeros(B, dtype=torch.long)
        for _ in range(3):
            v = 2 * v + 1 + (x[torch.arange(B), ord_[tree][v]] - thr[tree][v] > 0).long()
        return v - 7

    purities = []
    for tree in range(T):
        leaf = leaves(tree)
        purities.append(sum(int(torch.bincount(y[leaf == k], minlength=4).max()) for k in range(8)) / B)
        closed = thr[tree] == torch.finfo(torch.float32).max          # a vertex that could not be split
        for v in closed.nonzero().flatten().tolist():
            assert v > 0 and ord_[tree][v] == ord_[tree][(v - 1) // 2]
        root_values = x[:, ord_[tree][0]].sort().values               # a threshold is a midpoint of two data values
        assert (((root_values[1:] + root_values[:-1]) / 2 - thr[tree][0]).abs() < 1e-6).any()
    majority = int(torch.bincount(y).max()) / B
    assert min(purities) > majority + 0.2 and max(purities) > 0.95

    before = thr.clone()
    assert hingetree_cpp.tree_init_greedy(x, torch.zeros(B, dtype=torch.long), thr, ord_, w) is False  # one class
    assert hingetree_cpp.tree_init_greedy(x, -y, thr, ord_, w) is False                                # negative labels
    assert hingetree_cpp.tree_init_greedy(x, y.float(), thr, ord_, w) is False                         # regression labels
    assert torch.equal(thr, before)
    with pytest.raises(ValueError):
        hingetree_cpp.tree_init_greedy(x, y.int(), thr, ord_, w)
    assert R.RandomHingeForest(C, 4, 3).init_greedy(x, y) is True
