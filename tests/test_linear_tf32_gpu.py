"""The tensor-core projection (ht_linear_tf32_stats_f32) and the LinearBatchNorm1d module built on it.

Bars: z = x w^T is computed with TF32 products (the tensor core reads the upper 19 bits of each fp32 operand) and
fp32 accumulation: |z - exact| <= 2e-3 * sum_k |x||w| per element, the tolerance BASELINE's configuration 5 allows
for its Linear.  The column sums and sums of squares are sums of the z that was written: 1e-5 relative to the
summed magnitudes.  The module matches torch.nn.Linear (fp32) + torch.nn.BatchNorm1d within the same TF32 bar on
the normalised scale, and its gradients match autograd through the torch modules within 1e-2 of the largest
gradient (TF32 in the forward, torch's matmul in the backward).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(128, 128, 32), (300, 260, 100), (77, 12, 8), (1024, 1200, 784), (8192, 12700, 784)],
                         ids=str)
def test_projection_and_statistics(shape):
    from hingetreefortorch_b200 import _cabi
    M, N, K = shape
    gen = torch.Generator(device="cuda").manual_seed(M + N + K)
    x = torch.rand((M, K), device="cuda", generator=gen)
    w = (torch.rand((N, K), device="cuda", generator=gen) - 0.5) / K ** 0.5
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    z, total, total_sq = _cabi.linear_tf32_stats(x, w, status)
    assert int(status.item()) == 0
    exact = x.double() @ w.double().t()
    scale = x.abs().double() @ w.abs().double().t()
    assert bool(((z.double() - exact).abs() <= 2e-3 * scale).all())
    zd = z.double()
    assert bool(((total.double() - zd.sum(0)).abs() <= 1e-5 * zd.abs().sum(0) + 1e-30).all())
    assert bool(((total_sq.double() - (zd * zd).sum(0)).abs() <= 1e-5 * (zd * zd).sum(0) + 1e-30).all())
    again = _cabi.linear_tf32_stats(x, w, status)[0]
    assert torch.equal(z, again)  # the product itself has a fixed summation order


def test_projection_rejects_rows_that_are_not_16_byte_multiples():
    from hingetreefortorch_b200 import _cabi
    x, w = torch.zeros(8, 6, device="cuda"), torch.zeros(8, 6, device="cuda")
    with pytest.raises(_cabi.HingeTreeError) as err:
        _cabi.linear_tf32_stats(x, w)
    assert err.value.status == -5


def test_linear_batchnorm_module_against_torch():
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(11)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ours = R.LinearBatchNorm1d(64, 128).cuda()
        lin = torch.nn.Linear(64, 128, bias=False).cuda()
        bn = torch.nn.BatchNorm1d(128, affine=False).cuda()
        with torch.no_grad():
            lin.weight.copy_(ours.weight)
        x = torch.rand(512, 64, device="cuda")
        g = torch.randn(512, 128, device="cuda")
        y = ours(x)
        ref = bn(lin(x))
        assert float((y - ref).detach().abs().max()) <= 2e-2  # normalised activations are O(1); TF32 products upstream
        assert torch.allclose(ours.running_mean, bn.running_mean, atol=1e-3)
        assert torch.allclose(ours.running_var, bn.running_var, rtol=1e-2, atol=1e-4)
        assert int(ours.num_batches_tracked) == 1
        (y * g).sum().backward()
        (ref * g).sum().backward()
        scale = float(lin.weight.grad.abs().max())
        assert float((ours.weight.grad - lin.weight.grad).abs().max()) <= 1e-2 * scale
        ours.eval()
        bn.eval()
        assert float((ours(x) - bn(lin(x))).detach().abs().max()) <= 2e-2
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_pipeline_of_the_reference_readme_runs_on_the_module():
    """Linear -> BatchNorm -> sequential-initialisation forest, the forest stage exact given its input."""
    from hingetreefortorch_b200 import RandomHingeForest as R
    from oracle import hinge_oracle as ho
    torch.manual_seed(12)
    trees, depth = 12, 5
    hidden = trees * (2 ** depth - 1) + 4 - (trees * (2 ** depth - 1)) % 4 if (trees * (2 ** depth - 1)) % 4 else trees * (2 ** depth - 1)
    front = R.LinearBatchNorm1d(40, hidden).cuda()
    forest = R.RandomHingeForest(hidden, trees, depth, init_type="sequential").cuda()
    x = torch.rand(256, 40, device="cuda")
    z = front(x)
    y = forest(z)
    y.sum().backward()
    want = ho.forward("tree", z.detach().cpu().numpy(), forest.thresholds.detach().cpu().numpy(),
                      forest.ordinals.cpu().numpy(), forest.weights.detach().cpu().numpy())
    assert np.array_equal(y.detach().cpu().numpy(), want)
    assert front.weight.grad is not None and bool(torch.isfinite(front.weight.grad).all())


@pytest.mark.parametrize("kind", ["tree", "fern"])
@pytest.mark.parametrize("extra", [(), (3,)])
def test_forest_on_unmaterialised_normalisation(kind, extra):
    """`*_normalised_forward` on raw activations equals the plain forward on ATen's materialised normalisation bit for
    bit; `*_normalised_backward` gives the forest's parameter gradients at the usual bar and, for the gradient with
    respect to the raw activations, what torch's batch-norm backward makes of the plain backward's dense gradient."""
    from conftest import grad_close
    from hingetreefortorch_b200._ext import hingetree_cpp as ext
    from oracle import hinge_oracle as ho
    gen = torch.Generator().manual_seed(5)
    B, C, T, depth = 300, 52, 11, 5
    N = depth if kind == "fern" else 2 ** depth - 1
    z = (torch.randn(B, C, generator=gen) * 3 + 1).cuda()
    thr = (torch.rand(T, N, generator=gen) * 2 - 1).cuda()
    ord_ = torch.randint(0, C, (T, N), generator=gen).cuda()
    w = torch.randn((T, 2 ** depth) + extra, generator=gen).cuda()
    g = torch.randn((B, T) + extra, generator=gen).cuda()
    mean = z.mean(0)
    invstd = torch.rsqrt(z.var(0, unbiased=False) + 1e-5)
    y = torch.batch_norm_elemt(z, None, None, mean, invstd, 1e-5)
    plain = getattr(ext, kind + "_forward")(y, thr, ord_, w)
    fused, no_margin, no_where = getattr(ext, kind + "_normalised_forward")(z, mean, invstd, thr, ord_, w)
    assert torch.equal(fused, plain) and no_margin.numel() == 0 and no_where.numel() == 0
    kept_out, margin, where = getattr(ext, kind + "_normalised_forward")(z, mean, invstd, thr, ord_, w, True)
    assert torch.equal(kept_out, plain) and margin.shape == (B, T) and where.shape == (B, T, 2)
    dz, gthr, gw = getattr(ext, kind + "_normalised_backward")(z, mean, invstd, thr, True, ord_, w, True, g)
    kept = getattr(ext, kind + "_normalised_backward")(z, mean, invstd, thr, True, ord_, w, True, g, margin, where)
    want = ho.backward(kind, y.cpu().numpy(), thr.cpu().numpy(), ord_.cpu().numpy(), w.cpu().numpy(), g.cpu().numpy())
    mags = ho.backward_magnitudes(kind, y.cpu().numpy(), thr.cpu().numpy(), ord_.cpu().numpy(), w.cpu().numpy(), g.cpu().numpy())
    assert grad_close(gthr, want[1], mags[1]) and grad_close(gw, want[2], mags[2])
    gy = torch.from_numpy(want[0]).cuda()  # dense gradient with respect to the normalised activations
    sum_dy, sum_dy_xmu, _, _ = torch.batch_norm_backward_reduce(gy, z, mean, invstd, None, True, False, False)
    count = torch.full((1,), B, dtype=torch.int32, device="cuda")
    want_dz = torch.batch_norm_backward_elemt(gy, z, mean, invstd, None, sum_dy, sum_dy_xmu, count)
    scale = float(want_dz.abs().max())
    assert float((dz - want_dz).abs().max()) <= 2e-5 * scale
    # from the kept traversal: the same parameter gradients (same terms; sums in free order), the same dz to a rounding
    assert grad_close(kept[1], want[1], mags[1]) and grad_close(kept[2], want[2], mags[2])
    assert float((kept[0] - want_dz).abs().max()) <= 2e-5 * scale
    only = getattr(ext, kind + "_normalised_backward")(z, mean, invstd, thr, False, ord_, w, False, g)
    assert only[1] is None and only[2] is None and float((only[0] - want_dz).abs().max()) <= 2e-5 * scale


def test_fused_front_and_forest_module_against_the_pair():
    """LinearBatchNormForest in training mode against its own two modules run one after the other on the same
    parameters: outputs equal bit for bit (same z, same statistics, same rounding of the normalisation), gradients
    within the tolerance of sums in another order; running statistics advance the same way; evaluation mode is the pair."""
    from hingetreefortorch_b200 import RandomHingeForest as R
    torch.manual_seed(13)
    trees, depth, hidden = 12, 5, 372  # 12 * 31
    pair_front = R.LinearBatchNorm1d(40, hidden).cuda()
    pair_forest = R.RandomHingeForest(hidden, trees, depth, init_type="sequential").cuda()
    front, forest = R.LinearBatchNorm1d(40, hidden).cuda(), R.RandomHingeForest(hidden, trees, depth, init_type="sequential").cuda()
    front.load_state_dict(pair_front.state_dict())
    forest.load_state_dict(pair_forest.state_dict())
    fused = R.LinearBatchNormForest(front, forest)
    x = torch.rand(256, 40, device="cuda")
    out = fused(x)
    ref = pair_forest(pair_front(x))
    assert torch.equal(out, ref)
    g = torch.randn_like(out)
    (out * g).sum().backward()
    (ref * g).sum().backward()
    for a, b in ((front.weight.grad, pair_front.weight.grad), (forest.thresholds.grad, pair_forest.thresholds.grad),
                 (forest.weights.grad, pair_forest.weights.grad)):
        assert float((a - b).abs().max()) <= 1e-3 * float(b.abs().max()) + 1e-6
    assert torch.equal(front.running_mean, pair_front.running_mean) and torch.equal(front.running_var, pair_front.running_var)
    fused.eval(), pair_front.eval(), pair_forest.eval()
    assert torch.equal(fused(x), pair_forest(pair_front(x)))
