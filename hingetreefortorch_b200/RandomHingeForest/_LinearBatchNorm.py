"""Linear (no bias) followed by BatchNorm1d(affine=False) as one module on the tensor cores.

This is the front of the reference's sequential-initialisation pipeline (README.md:110-129:
``nn.Linear(in, trees * (2**depth - 1), bias=False)`` -> ``nn.BatchNorm1d(..., affine=False)`` ->
``RandomHingeForest(..., init_type="sequential")``), which the reference builds from torch modules.
Here the projection runs as a TF32 tensor-core kernel of this library whose epilogue also produces the
per-column sums and sums of squares of the activations, so batch normalisation does not read the
activations again for its statistics.  Parameter and buffer names are those of nn.Linear / nn.BatchNorm1d
(``weight``, ``running_mean``, ``running_var``, ``num_batches_tracked``).
"""
import math

import torch
import torch.nn as nn

from .._ext import hingetree_cpp


class _LinearBatchNorm(torch.autograd.Function):
    """y = (z - mean) * invstd with z = x @ w.T (TF32 products, fp32 accumulation) and mean / invstd either the batch
    statistics of z, which come out of the projection kernel's epilogue, or given ones.

    The normalisation and its backward use ATen's fused element-wise and reduction kernels for batch normalisation
    (the ones torch.nn.SyncBatchNorm is built from), so the activations are read once in the forward and twice in
    the backward.  The weight (and input) gradients are products of the same size as the forward's and are taken in
    TF32 as well, by torch.matmul."""

    @staticmethod
    def forward(ctx, x, w, eps, given_mean, given_var):
        x, w = x.contiguous(), w.contiguous()
        z, total, total_sq = hingetree_cpp.linear_tf32_stats(x, w)
        rows = x.shape[0]
        if given_mean is None:
            mean, var, invstd = hingetree_cpp.batchnorm_statistics(total, total_sq, rows, eps)
        else:
            mean, var = given_mean, given_var
            invstd = torch.rsqrt(var + eps)
        y = torch.batch_norm_elemt(z, None, None, mean, invstd, eps)
        ctx.batch_statistics = given_mean is None
        ctx.save_for_backward(x, w, z, mean, invstd)
        ctx.mark_non_differentiable(mean, var)
        return y, mean, var

    @staticmethod
    def backward(ctx, grad_y, _grad_mean, _grad_var):
        x, w, z, mean, invstd = ctx.saved_tensors
        grad_y = grad_y.contiguous()
        if ctx.batch_statistics:
            sum_dy, sum_dy_xmu, _, _ = torch.batch_norm_backward_reduce(grad_y, z, mean, invstd, None, True, False, False)
            count = torch.full((1,), z.shape[0], dtype=torch.int32, device=z.device)
            grad_z = torch.batch_norm_backward_elemt(grad_y, z, mean, invstd, None, sum_dy, sum_dy_xmu, count)
        else:
            grad_z = grad_y * invstd
        previous = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            grad_x = grad_z @ w if ctx.needs_input_grad[0] else None
            grad_w = grad_z.t() @ x if ctx.needs_input_grad[1] else None
        finally:
            torch.backends.cuda.matmul.allow_tf32 = previous
        return grad_x, grad_w, None, None, None


class LinearBatchNorm1d(nn.Module):
    """y = BatchNorm1d(affine=False)(x @ weight.T): training mode normalises with the batch statistics (biased
    variance) and updates the running ones (unbiased variance, as nn.BatchNorm1d does); evaluation mode uses the
    running statistics.  in_features and out_features must be multiples of 4."""

    def __init__(self, in_features, out_features, eps=1e-5, momentum=0.1):
        super().__init__()
        if in_features % 4 or out_features % 4:
            raise ValueError("in_features and out_features must be multiples of 4")
        self.in_features, self.out_features, self.eps, self.momentum = in_features, out_features, eps, momentum
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        nn.init.kaiming_uniform_(self.weight, a=math.sqrt(5))  # nn.Linear's default
        self.register_buffer("running_mean", torch.zeros(out_features))
        self.register_buffer("running_var", torch.ones(out_features))
        self.register_buffer("num_batches_tracked", torch.tensor(0, dtype=torch.long))

    def forward(self, x):
        if not self.training:
            return _LinearBatchNorm.apply(x, self.weight, self.eps, self.running_mean, self.running_var)[0]
        y, mean, var = _LinearBatchNorm.apply(x, self.weight, self.eps, None, None)
        with torch.no_grad():
            rows = x.shape[0]
            self.num_batches_tracked += 1
            self.running_mean.lerp_(mean, self.momentum)
            self.running_var.lerp_(var * (rows / max(rows - 1, 1)), self.momentum)
        return y

    def extra_repr(self):
        return "in_features=%d, out_features=%d, eps=%g, momentum=%g" % (self.in_features, self.out_features, self.eps,
                                                                         self.momentum)


class _LinearBatchNormForest(torch.autograd.Function):
    """forest((z - mean) * invstd) with z = x @ w.T and batch statistics, the normalised activations never written:
    the forest normalises the features it visits (bit-identical to the forest behind a materialised normalisation),
    and its backward hands the normalisation's backward a gradient of one entry per (sample, tree) and the two column
    sums it needs, so the gradient with respect to z takes one pass over z."""

    @staticmethod
    def forward(ctx, x, w, thresholds, ordinals, weights, eps, fern):
        x, w = x.contiguous(), w.contiguous()
        z, total, total_sq = hingetree_cpp.linear_tf32_stats(x, w)
        rows = x.shape[0]
        mean, var, invstd = hingetree_cpp.batchnorm_statistics(total, total_sq, rows, eps)
        op = hingetree_cpp.fern_normalised_forward if fern else hingetree_cpp.tree_normalised_forward
        out, margin, where = op(z, mean, invstd, thresholds, ordinals, weights, True)  # the traversal is kept
        ctx.fern = fern
        ctx.save_for_backward(x, w, z, mean, invstd, thresholds, ordinals, weights, margin, where)
        ctx.mark_non_differentiable(mean, var)
        return out, mean, var

    @staticmethod
    def backward(ctx, grad_out, _grad_mean, _grad_var):
        x, w, z, mean, invstd, thresholds, ordinals, weights, margin, where = ctx.saved_tensors
        op = hingetree_cpp.fern_normalised_backward if ctx.fern else hingetree_cpp.tree_normalised_backward
        grad_z, grad_thr, grad_weights = op(z, mean, invstd, thresholds, ctx.needs_input_grad[2], ordinals, weights,
                                            ctx.needs_input_grad[4], grad_out.contiguous(), margin, where)
        previous = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = True
        try:
            grad_x = grad_z @ w if ctx.needs_input_grad[0] else None
            grad_w = grad_z.t() @ x if ctx.needs_input_grad[1] else None
        finally:
            torch.backends.cuda.matmul.allow_tf32 = previous
        return grad_x, grad_w, grad_thr, None, grad_weights, None, None


class LinearBatchNormForest(nn.Module):
    """A LinearBatchNorm1d front and a RandomHingeForest / RandomHingeFern behind it as one step: in training mode the
    normalised activations are never materialised (see _LinearBatchNormForest); in evaluation mode the two modules
    run one after the other.  The parameters stay those of the two modules (``front.weight``, ``forest.thresholds``,
    ``forest.ordinals``, ``forest.weights``), so checkpoints of the unfused pair load as they are."""

    def __init__(self, front, forest):
        super().__init__()
        if not isinstance(front, LinearBatchNorm1d):
            raise TypeError("front must be a LinearBatchNorm1d")
        if forest.in_channels != front.out_features:
            raise ValueError("the forest reads %d channels, the front produces %d" % (forest.in_channels, front.out_features))
        self.front, self.forest = front, forest

    def forward(self, x):
        if not self.training:
            return self.forest(self.front(x))
        front, forest = self.front, self.forest
        out, mean, var = _LinearBatchNormForest.apply(x, front.weight, forest.thresholds, forest.ordinals, forest.weights,
                                                      front.eps, bool(forest._fern))
        with torch.no_grad():
            rows = x.shape[0]
            front.num_batches_tracked += 1
            front.running_mean.lerp_(mean, front.momentum)
            front.running_var.lerp_(var * (rows / max(rows - 1, 1)), front.momentum)
        return out
