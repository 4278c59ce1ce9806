"""nn.Module layer: random hinge forests, ferns and their fused-linear / fusion / sparse variants.

Constructor arguments, parameter names (`weights`, `thresholds`, `ordinals`, `linear_weights`,
`linear_bias`), parameter shapes and the order in which the random number generator is
consumed (thresholds, then ordinals, then weights) follow the reference's
RandomHingeForest/_RandomHingeForest.py, so that a seeded construction yields the same
parameters and its checkpoints load unchanged.
"""
import math

import torch
import torch.nn as nn
import torch.nn.init as init

from .. import HingeTree as _F


def _thresholds(out_channels, decisions):
    return 6.0 * torch.rand([out_channels, decisions]) - 3.0


def _sequential_ordinals(like, in_channels):
    ordinals = torch.arange(like.numel(), dtype=torch.long)
    return (ordinals % in_channels).reshape(like.shape)


def _leaf_weights(out_channels, leaves, extra_outputs):
    if extra_outputs is None:
        return torch.randn([out_channels, leaves])
    if hasattr(extra_outputs, "__iter__"):
        return torch.randn([out_channels, leaves] + list(extra_outputs))
    return torch.randn([out_channels, leaves, extra_outputs])


class _HingeBase(nn.Module):
    """Parameters and analysis helpers shared by forests and ferns.

    Subclasses set `_function` (the autograd Function), `_fern` and, for ferns, nothing else:
    a tree has 2**depth - 1 decisions, a fern has `depth`.
    """
    __constants__ = ["in_channels", "out_channels", "depth", "extra_outputs", "init_type"]
    _function = None
    _fern = False

    def __init__(self, in_channels: int, out_channels: int, depth: int, extra_outputs=None, init_type: str = "random"):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.depth = depth
        self.extra_outputs = extra_outputs
        self.init_type = init_type

        thresholds = _thresholds(out_channels, self._decisions(depth))
        ordinals = self._init_ordinals(thresholds, in_channels, init_type)
        weights = _leaf_weights(out_channels, self._weight_rows(depth), extra_outputs)
        self._hygiene(thresholds, ordinals, weights)

        self.weights = nn.Parameter(weights, requires_grad=True)
        self.thresholds = nn.Parameter(thresholds, requires_grad=True)
        self.ordinals = nn.Parameter(ordinals, requires_grad=False)

    @classmethod
    def _decisions(cls, depth):
        return depth if cls._fern else 2 ** depth - 1

    @classmethod
    def _weight_rows(cls, depth):
        return 2 ** depth

    def _init_ordinals(self, thresholds, in_channels, init_type):
        if init_type == "random":
            return torch.randint_like(thresholds, low=0, high=in_channels, dtype=torch.long)
        if init_type == "sequential":
            return _sequential_ordinals(thresholds, in_channels)
        raise RuntimeError(f"Unknown init_type {init_type}. Must be one of 'random' or 'sequential'.")

    def _hygiene(self, thresholds, ordinals, weights):
        self._function.fix_thresholds(thresholds, ordinals, weights)

    def _params(self):
        return self.thresholds, self.ordinals, self.weights

    def forward(self, x):
        return self._function.apply(x, *self._params())

    def reachability(self, x):
        return self._function.reachability(x, *self._params())

    def leafmap(self, x):
        return self._function.leafmap(x, *self._params())

    def marginmap(self, x):
        return self._function.marginmap(x, *self._params())

    def check_thresholds(self):
        return self._function.check_thresholds(self.thresholds.data, self.ordinals.data, self.weights.data)

    def fix_thresholds(self):
        return self._function.fix_thresholds(self.thresholds.data, self.ordinals.data, self.weights.data)

    def init_medians(self, x):
        return self._function.init_medians(x, self.thresholds.data, self.ordinals.data, self.weights.data)

    def load_state_dict(self, *args, **kwargs):
        result = super().load_state_dict(*args, **kwargs)
        # old checkpoints store the ordinals as float32
        self.ordinals = nn.Parameter(self.ordinals.data.type(torch.long), requires_grad=False)
        return result


class RandomHingeForest(_HingeBase):
    _function = _F.HingeTree

    def pathmap(self, x):
        """Feature indices on the root-to-leaf path of heap leaf `leaf key`, per sample: [..., depth].

        Follows the reference's arithmetic (_RandomHingeForest.py:88-121): the leaf key is taken
        as the rank of a leaf in heap order and its ancestors are listed root first.
        """
        leaf = self.leafmap(x)
        shape = list(leaf.shape)
        leaf = leaf.reshape(shape[0], shape[1], -1)
        trees = torch.arange(shape[1], device=leaf.device).view(1, -1, 1)
        vertex = leaf + (2 ** self.depth - 1)
        steps = [None] * self.depth
        for level in reversed(range(self.depth)):
            vertex = torch.div(vertex - 1, 2, rounding_mode="floor")
            steps[level] = self.ordinals[trees, vertex]
        return torch.stack(steps, dim=-1).view(shape + [self.depth])

    def init_greedy(self, x, y):
        return _F.HingeTree.init_greedy(x, y, self.thresholds.data, self.ordinals.data, self.weights.data)


class RandomHingeFern(_HingeBase):
    _function = _F.HingeFern
    _fern = True

    def pathmap(self, x):
        """Every fern tests all of its features: the path map is the ordinals, broadcast over samples."""
        if x.dim() < 2:
            raise RuntimeError("Input batch should be at least 2 dimensions.")
        ordinals = self.ordinals.view([1, self.out_channels] + [1] * (x.dim() - 2) + [self.depth])
        return ordinals.expand([x.shape[0], self.out_channels] + list(x.shape[2:]) + [self.depth]).contiguous()


class RandomHingeTrie(_HingeBase):
    """Weights sit on the internal vertices; every decision on the path contributes."""
    _function = _F.HingeTrie

    @classmethod
    def _weight_rows(cls, depth):
        return 2 ** depth - 1

    def _hygiene(self, thresholds, ordinals, weights):
        pass


class SparseRandomHingeForest(RandomHingeForest):
    _function = _F.SparseHingeTree


class SparseRandomHingeFern(RandomHingeFern):
    _function = _F.SparseHingeFern


class _FusedLinearMixin:
    """Adds the [out_channels, number_of_trees] linear layer applied to the tree outputs."""

    def _init_linear(self, number_of_trees, out_channels, bias):
        self.linear_weights = nn.Parameter(torch.empty([out_channels, number_of_trees]))
        self.linear_bias = nn.Parameter(torch.zeros([out_channels]), requires_grad=bias)
        init.kaiming_uniform_(self.linear_weights, a=math.sqrt(5))
        if bias:
            fan_in, _ = init._calculate_fan_in_and_fan_out(self.linear_weights)
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            init.uniform_(self.linear_bias, -bound, bound)

    def _params(self):
        return self.thresholds, self.ordinals, self.weights, self.linear_weights, self.linear_bias


class RandomHingeForestFusedLinear(_FusedLinearMixin, RandomHingeForest):
    _linear_function = _F.HingeTreeFusedLinear

    def __init__(self, in_channels: int, number_of_trees: int, out_channels: int, depth: int, extra_outputs=None,
                 init_type: str = "random", bias: bool = True):
        super().__init__(in_channels, number_of_trees, depth, extra_outputs, init_type)
        self._init_linear(number_of_trees, out_channels, bias)

    def forward(self, x):
        return self._linear_function.apply(x, *self._params())

    def _tree_params(self):
        return self.thresholds, self.ordinals, self.weights

    def reachability(self, x):
        return self._function.reachability(x, *self._tree_params())

    def leafmap(self, x):
        return self._function.leafmap(x, *self._tree_params())

    def marginmap(self, x):
        return self._function.marginmap(x, *self._tree_params())


class RandomHingeFernFusedLinear(_FusedLinearMixin, RandomHingeFern):
    _linear_function = _F.HingeFernFusedLinear

    def __init__(self, in_channels: int, number_of_trees: int, out_channels: int, depth: int, extra_outputs=None,
                 init_type: str = "random", bias: bool = True):
        super().__init__(in_channels, number_of_trees, depth, extra_outputs, init_type)
        self._init_linear(number_of_trees, out_channels, bias)

    forward = RandomHingeForestFusedLinear.forward
    _tree_params = RandomHingeForestFusedLinear._tree_params
    reachability = RandomHingeForestFusedLinear.reachability
    leafmap = RandomHingeForestFusedLinear.leafmap
    marginmap = RandomHingeForestFusedLinear.marginmap


class SparseRandomHingeForestFusedLinear(RandomHingeForestFusedLinear):
    _linear_function = _F.SparseHingeTreeFusedLinear


class SparseRandomHingeFernFusedLinear(RandomHingeFernFusedLinear):
    _linear_function = _F.SparseHingeFernFusedLinear


class _FusionBase(_HingeBase):
    """Trees over the concatenation of image channels and a per-sample feature vector."""
    __constants__ = ["img_channels", "vec_channels", "out_channels", "depth", "extra_outputs", "init_type"]
    _fusion_function = None

    def __init__(self, img_channels: int, vec_channels: int, out_channels: int, depth: int, extra_outputs=None,
                 init_type: str = "balanced_random", p=0.5):
        self._p = p
        self._split = (img_channels, vec_channels)
        super().__init__(img_channels + vec_channels, out_channels, depth, extra_outputs, init_type)
        self.img_channels = img_channels
        self.vec_channels = vec_channels
        del self.in_channels

    def _init_ordinals(self, thresholds, in_channels, init_type):
        if init_type == "balanced_random":
            p = self._p
            img_channels, vec_channels = self._split
            assert 0.0 <= p <= 1.0
            # a feature is drawn from the image with probability p and from the vector otherwise
            feature_weights = [p / img_channels] * img_channels + [(1.0 - p) / vec_channels] * vec_channels
            drawn = list(torch.utils.data.WeightedRandomSampler(feature_weights, thresholds.numel(), replacement=True))
            return torch.tensor(drawn, dtype=torch.long).view(thresholds.shape)
        return super()._init_ordinals(thresholds, in_channels, init_type)

    def forward(self, img, vec):
        assert img.shape[1] == self.img_channels and vec.shape[1] == self.vec_channels
        return self._fusion_function.apply(img, vec, *self._params())


class RandomHingeForestFusion(_FusionBase):
    _function = _F.HingeTree
    _fusion_function = _F.HingeTreeFusion


class RandomHingeFernFusion(_FusionBase):
    _function = _F.HingeFern
    _fusion_function = _F.HingeFernFusion
    _fern = True


class RandomHingeForestFusionFusedLinear(_FusedLinearMixin, RandomHingeForestFusion):
    _fusion_function = _F.HingeTreeFusionFusedLinear

    def __init__(self, img_channels: int, vec_channels: int, number_of_trees: int, out_channels: int, depth: int,
                 extra_outputs=None, init_type: str = "balanced_random", p=0.5, bias: bool = True):
        super().__init__(img_channels, vec_channels, number_of_trees, depth, extra_outputs, init_type, p)
        self._init_linear(number_of_trees, out_channels, bias)


class RandomHingeFernFusionFusedLinear(_FusedLinearMixin, RandomHingeFernFusion):
    _fusion_function = _F.HingeFernFusionFusedLinear

    def __init__(self, img_channels: int, vec_channels: int, number_of_trees: int, out_channels: int, depth: int,
                 extra_outputs=None, init_type: str = "balanced_random", p=0.5, bias: bool = True):
        super().__init__(img_channels, vec_channels, number_of_trees, depth, extra_outputs, init_type, p)
        self._init_linear(number_of_trees, out_channels, bias)
