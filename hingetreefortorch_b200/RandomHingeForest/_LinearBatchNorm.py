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


class _LinearStats(torch.autograd.Function):
    """(z, sum_m z, sum_m z*z) = f(x, w) with z = x @ w.T; TF32 products, fp32 accumulation."""

    @staticmethod
    def forward(ctx, x, w):
        z, total, total_sq = hingetree_cpp.linear_tf32_stats(x.contiguous(), w.contiguous())
        ctx.save_for_backward(x, w, z)
        return z, total, total_sq

    @staticmethod
    def backward(ctx, grad_z, grad_total, grad_total_sq):
        x, w, z = ctx.saved_tensors
        g = grad_z
        if grad_total is not None:
            g = g + grad_total.unsqueeze(0)
        if grad_total_sq is not None:
            g = torch.addcmul(g, z, grad_total_sq.unsqueeze(0), value=2.0)
        grad_x = g @ w if ctx.needs_input_grad[0] else None
        grad_w = g.t() @ x if ctx.needs_input_grad[1] else None
        return grad_x, grad_w


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
        z, total, total_sq = _LinearStats.apply(x, self.weight)
        if self.training:
            rows = x.shape[0]
            mean = total / rows
            var = (total_sq / rows - mean * mean).clamp_min(0.0)
            with torch.no_grad():
                self.num_batches_tracked += 1
                unbiased = var * (rows / max(rows - 1, 1))
                self.running_mean.lerp_(mean.detach(), self.momentum)
                self.running_var.lerp_(unbiased.detach(), self.momentum)
        else:
            mean, var = self.running_mean, self.running_var
        return (z - mean) * torch.rsqrt(var + self.eps)

    def extra_repr(self):
        return "in_features=%d, out_features=%d, eps=%g, momentum=%g" % (self.in_features, self.out_features, self.eps,
                                                                         self.momentum)
