"""Convolutional hinge trees / ferns: one single-channel tree per (output channel, input channel).

Each tree looks at the kernel window of ONE input channel (ordinals index the window cells in
row-major order) and the contributions are summed over the input channels.  Constructor
arguments and parameter shapes follow the reference's RandomHingeForest/_HingeTreeConv.py:
thresholds and ordinals [out, in, decisions], weights [out, in, leaves(, extra_outputs)].
"""
from functools import reduce
import operator

import torch
import torch.nn as nn

from .. import HingeTree as _F


def _as_tuple(x, n: int):
    if isinstance(x, int):
        return (x,) * n
    if len(x) != n:
        raise RuntimeError(f"Expected size {n} list/tuple.")
    return tuple(x)


class _HingeConvBase(nn.Module):
    __constants__ = ["in_channels", "out_channels", "depth", "extra_outputs", "kernel_size", "stride", "padding",
                     "dilation", "init_type"]
    _dims = 2
    _fern = False
    _function = None
    _hygiene = None

    def __init__(self, in_channels: int, out_channels: int, depth: int, kernel_size, stride=1, padding=0, dilation=1,
                 extra_outputs: int = 1, init_type: str = "random"):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.depth = depth
        self.extra_outputs = extra_outputs
        self.init_type = init_type
        n = self._dims
        self.kernel_size = _as_tuple(kernel_size, n)
        self.stride = _as_tuple(stride, n)
        self.padding = _as_tuple(padding, n)
        self.dilation = _as_tuple(dilation, n)

        decisions = depth if self._fern else 2 ** depth - 1
        thresholds = 6.0 * torch.rand([out_channels, in_channels, decisions]) - 3.0
        window = reduce(operator.mul, self.kernel_size)
        if init_type == "random":
            ordinals = torch.randint_like(thresholds, low=0, high=window, dtype=torch.long)
        elif init_type == "sequential":
            ordinals = (torch.arange(thresholds.numel(), dtype=torch.long) % window).reshape(thresholds.shape)
        else:
            raise RuntimeError(f"Unknown init_type {init_type}. Must be one of 'random' or 'sequential'.")
        if extra_outputs > 1:
            weights = torch.randn([out_channels, in_channels, 2 ** depth, extra_outputs])
        else:
            weights = torch.randn([out_channels, in_channels, 2 ** depth])
        trees = out_channels * in_channels
        self._hygiene.fix_thresholds(thresholds.view([trees, -1]), ordinals.view([trees, -1]),
                                     weights.view([trees, 2 ** depth, -1]))
        self.weights = nn.Parameter(weights, requires_grad=True)
        self.thresholds = nn.Parameter(thresholds, requires_grad=True)
        self.ordinals = nn.Parameter(ordinals, requires_grad=False)

    def forward(self, x):
        return self._function.apply(x, self.thresholds, self.ordinals, self.weights, self.kernel_size, self.stride,
                                    self.padding, self.dilation)


def _conv_module(name, dims, fern):
    function = getattr(_F, "Hinge%sConv%dd" % ("Fern" if fern else "Tree", dims))
    hygiene = _F.HingeFern if fern else _F.HingeTree
    return type(name, (_HingeConvBase,), {"_dims": dims, "_fern": fern, "_function": function, "_hygiene": hygiene,
                                          "__module__": __name__})


HingeTreeConv1d = _conv_module("HingeTreeConv1d", 1, False)
HingeTreeConv2d = _conv_module("HingeTreeConv2d", 2, False)
HingeTreeConv3d = _conv_module("HingeTreeConv3d", 3, False)
HingeFernConv1d = _conv_module("HingeFernConv1d", 1, True)
HingeFernConv2d = _conv_module("HingeFernConv2d", 2, True)
HingeFernConv3d = _conv_module("HingeFernConv3d", 3, True)
