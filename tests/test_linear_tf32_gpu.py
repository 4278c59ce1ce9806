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
