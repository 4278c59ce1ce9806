"""torch.autograd.Function layer over the `hingetree_cpp` operators.

Class names, argument order and behaviour follow the reference's HingeTree/_HingeTree.py so
that model code written against it keeps working; the classes themselves are generated from a
few templates instead of being spelled out one by one.

Every Function saves its raw inputs and lets the backward operator redo the traversal, as the
reference does (_HingeTree.py:92-108); the plain tree and fern additionally keep the forward's
traversal where the library offers it, so that one training step walks the trees once.  Deterministic mode is read from
torch.are_deterministic_algorithms_enabled() (reference: _HingeTree.py:24-30): the plain tree
and fern select the fixed-order backward; operators without a fixed-order implementation
raise RuntimeError, as the reference does for every GPU operator other than the plain ones.
"""
import torch

from .._ext import hingetree_cpp


def _is_deterministic():
    """Whether torch is in deterministic mode, under whichever name this torch has for the query."""
    for query in ("are_deterministic_algorithms_enabled", "is_deterministic"):
        fn = getattr(torch, query, None)
        if fn is not None:
            return bool(fn())
    raise RuntimeError("Unable to query torch deterministic mode.")


def _op(name):
    return getattr(hingetree_cpp, name)


def _refuse_deterministic(tensor, what):
    if _is_deterministic() and tensor.device.type != "cpu":
        raise RuntimeError("No deterministic implementation of %s on GPUs." % what)


def _interleave(tensors, flags):
    """(t0, need0, t1, need1, ...) as the backward operators take them."""
    args = []
    for t, f in zip(tensors, flags):
        args += [t, f]
    return args


# ---- contract / expand ---------------------------------------------------------------------
# contract: [B, C, *image] -> [B, C, *windows, *window] (non-overlapping windows); expand is its inverse, and each is
# the other's gradient (the reference: _HingeTree.py:32-89).  A scalar window or padding applies to every dimension.

def _per_dimension(value, count):
    return [value] * count if isinstance(value, int) else value


def contract(inData, window, padding=0):
    dims = inData.dim() - 2
    return hingetree_cpp.contract(inData, _per_dimension(window, dims), _per_dimension(padding, dims))


def expand(inData, padding=0):
    return hingetree_cpp.expand(inData, _per_dimension(padding, (inData.dim() - 2) // 2))


class _Patches(torch.autograd.Function):
    """Both directions as one Function: `window` given means contract, None means expand; the backward runs the
    other direction with the window the forward saw."""

    @staticmethod
    def forward(ctx, inData, window, padding):
        ctx.padding = padding
        if window is None:
            dims = (inData.dim() - 2) // 2
            ctx.window = list(inData.shape[-dims:])
            return expand(inData, padding)
        ctx.window = None
        return contract(inData, window, padding)

    @staticmethod
    def backward(ctx, outDataGrad):
        if not ctx.needs_input_grad[0]:
            return None, None, None
        grad = outDataGrad.contiguous()
        if ctx.window is None:
            return expand(grad, ctx.padding), None, None
        return contract(grad, ctx.window, ctx.padding), None, None


class _Expand:
    """The reference's name for the expand Function (`_Expand.apply(x, padding)`)."""

    @staticmethod
    def apply(inData, padding):
        return _Patches.apply(inData, None, padding)


class _Contract:
    """The reference's name for the contract Function (`_Contract.apply(x, window, padding)`)."""

    @staticmethod
    def apply(inData, window, padding=0):
        return _Patches.apply(inData, window, padding)


class Contract(torch.nn.Module):
    def __init__(self, window, padding=0):
        super().__init__()
        self.window, self.padding = window, padding

    def forward(self, inData):
        return _Patches.apply(inData, self.window, self.padding)


class Expand(torch.nn.Module):
    def __init__(self, padding=0):
        super().__init__()
        self.padding = padding

    def forward(self, inData):
        return _Patches.apply(inData, None, self.padding)


# ---- Function templates --------------------------------------------------------------------

_UTILITIES = ("check_thresholds", "fix_thresholds", "reachability", "leafmap", "marginmap", "init_medians")


def _utilities(kind):
    """The analysis / initialisation helpers the reference hangs on HingeTree and HingeFern."""
    members = {}
    for util in _UTILITIES:
        members[util] = staticmethod(_op("%s_%s" % (kind, util)))
    members["speedtest"] = staticmethod(lambda inData, _f=_op(kind + "_speedtest"): _f(inData, _is_deterministic()))
    if kind == "tree":
        members["init_greedy"] = staticmethod(hingetree_cpp.tree_init_greedy)
    return members


def _plain_function(name, kind):
    fwd, bwd, bwd_det = _op(kind + "_forward"), _op(kind + "_backward"), _op(kind + "_backward_deterministic")
    fwd_saving, bwd_saved = _op(kind + "_forward_saving"), _op(kind + "_backward_saved")

    def forward(ctx, inData, inThresholds, inOrdinals, inWeights):
        # When a gradient will be asked for, the forward keeps its traversal (signed margin, deciding vertex and
        # leaf of every evaluation) so that the backward does not walk the trees again; the operator returns an
        # empty `kept` for problems it does not do this for, and the backward then re-walks, as the reference does.
        kept = None
        if inData.is_cuda and any(ctx.needs_input_grad):
            out, kept = fwd_saving(inData, inThresholds, inOrdinals, inWeights)
            if kept.numel() == 0:
                kept = None
        else:
            out = fwd(inData, inThresholds, inOrdinals, inWeights)
        ctx.kept = kept
        ctx.save_for_backward(inData, inThresholds, inOrdinals, inWeights)
        return out

    def backward(ctx, outDataGrad):
        kept, ctx.kept = ctx.kept, None  # one backward per forward: the scratch is rewritten by it
        if kept is not None:
            return tuple(bwd_saved(*_interleave(ctx.saved_tensors, ctx.needs_input_grad), outDataGrad.contiguous(), kept,
                                   _is_deterministic()))
        op = bwd_det if _is_deterministic() else bwd
        return tuple(op(*_interleave(ctx.saved_tensors, ctx.needs_input_grad), outDataGrad.contiguous()))

    members = {"forward": staticmethod(forward), "backward": staticmethod(backward)}
    members.update(_utilities(kind))
    return type(name, (torch.autograd.Function,), members)


def _sparse_function(name, base, kind, label):
    """Backward returns sparse COO gradients; only the data gradient is densified (as in the reference)."""
    bwd = _op("sparse_%s_backward" % kind)

    fwd = _op(kind + "_forward")

    def forward(ctx, inData, inThresholds, inOrdinals, inWeights):  # the sparse backward has no use for a kept traversal
        ctx.save_for_backward(inData, inThresholds, inOrdinals, inWeights)
        return fwd(inData, inThresholds, inOrdinals, inWeights)

    def backward(ctx, outDataGrad):
        _refuse_deterministic(ctx.saved_tensors[0], "sparse hinge %s backward" % label)
        grads = list(bwd(*_interleave(ctx.saved_tensors, ctx.needs_input_grad), outDataGrad.contiguous()))
        if grads[0] is not None:
            grads[0] = grads[0].to_dense()
        return tuple(grads)

    return type(name, (base,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})


def _fused_linear_function(name, base, kind, label, sparse):
    fwd = _op(kind + "_fused_linear_forward")
    bwd = _op(("sparse_" if sparse else "") + kind + "_fused_linear_backward")

    def forward(ctx, inData, inThresholds, inOrdinals, inWeights, inLinearWeights, inLinearBias):
        _refuse_deterministic(inData, "forward for hinge %s + linear" % label)
        ctx.save_for_backward(inData, inThresholds, inOrdinals, inWeights, inLinearWeights, inLinearBias)
        return fwd(inData, inThresholds, inOrdinals, inWeights, inLinearWeights, inLinearBias)

    def backward(ctx, outDataGrad):
        _refuse_deterministic(outDataGrad, "backpropagation for hinge %s + linear" % label)
        grads = list(bwd(*_interleave(ctx.saved_tensors, ctx.needs_input_grad), outDataGrad.contiguous()))
        if sparse and grads[0] is not None:
            grads[0] = grads[0].to_dense()
        return tuple(grads)

    members = {"backward": staticmethod(backward)}
    if not sparse:
        members["forward"] = staticmethod(forward)
    return type(name, (base,), members)


def _fusion_function(name, kind, label):
    fwd, bwd = _op(kind + "_fusion_forward"), _op(kind + "_fusion_backward")

    def forward(ctx, inImg, inVec, inThresholds, inOrdinals, inWeights):
        ctx.save_for_backward(inImg, inVec, inThresholds, inOrdinals, inWeights)
        return fwd(inImg, inVec, inThresholds, inOrdinals, inWeights)

    def backward(ctx, outDataGrad):
        _refuse_deterministic(outDataGrad, "backpropagation for hinge %s fusion" % label)
        return tuple(bwd(*_interleave(ctx.saved_tensors, ctx.needs_input_grad), outDataGrad.contiguous()))

    return type(name, (torch.autograd.Function,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})


def _fusion_fused_linear_function(name, base, kind, label):
    fwd, bwd = _op(kind + "_fusion_fused_linear_forward"), _op(kind + "_fusion_fused_linear_backward")

    def forward(ctx, inImg, inVec, inThresholds, inOrdinals, inWeights, inLinearWeights, inLinearBias):
        _refuse_deterministic(inImg, "forward for hinge %s fusion + linear" % label)
        ctx.save_for_backward(inImg, inVec, inThresholds, inOrdinals, inWeights, inLinearWeights, inLinearBias)
        return fwd(inImg, inVec, inThresholds, inOrdinals, inWeights, inLinearWeights, inLinearBias)

    def backward(ctx, outDataGrad):
        # Returns the vector *gradient* in slot 1 (the reference returns the vector itself there for
        # trees and fails with a NameError for ferns, _HingeTree.py:345,362; neither is reproduced).
        _refuse_deterministic(outDataGrad, "backpropagation for hinge %s fusion + linear" % label)
        return tuple(bwd(*_interleave(ctx.saved_tensors, ctx.needs_input_grad), outDataGrad.contiguous()))

    return type(name, (base,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})


def _conv_function(name, kind, dims, label):
    fwd, bwd = _op("%s_conv%dd_forward" % (kind, dims)), _op("%s_conv%dd_backward" % (kind, dims))

    def forward(ctx, inData, inThresholds, inOrdinals, inWeights, kernelSize, stride, padding, dilation):
        ctx.save_for_backward(inData, inThresholds, inOrdinals, inWeights)
        ctx.geometry = (kernelSize, stride, padding, dilation)
        return fwd(inData, inThresholds, inOrdinals, inWeights, kernelSize, stride, padding, dilation)

    def backward(ctx, outDataGrad):
        _refuse_deterministic(outDataGrad, "backpropagation for hinge %s convolution" % label)
        grads = bwd(*_interleave(ctx.saved_tensors, ctx.needs_input_grad[:4]), outDataGrad.contiguous(), *ctx.geometry)
        return tuple(grads) + (None, None, None, None)

    return type(name, (torch.autograd.Function,), {"forward": staticmethod(forward), "backward": staticmethod(backward)})


HingeTree = _plain_function("HingeTree", "tree")
HingeFern = _plain_function("HingeFern", "fern")

SparseHingeTree = _sparse_function("SparseHingeTree", HingeTree, "tree", "tree")
SparseHingeFern = _sparse_function("SparseHingeFern", HingeFern, "fern", "fern")

HingeTreeFusedLinear = _fused_linear_function("HingeTreeFusedLinear", HingeTree, "tree", "tree", sparse=False)
HingeFernFusedLinear = _fused_linear_function("HingeFernFusedLinear", HingeFern, "fern", "fern", sparse=False)
SparseHingeTreeFusedLinear = _fused_linear_function("SparseHingeTreeFusedLinear", HingeTreeFusedLinear, "tree", "tree",
                                                    sparse=True)
SparseHingeFernFusedLinear = _fused_linear_function("SparseHingeFernFusedLinear", HingeFernFusedLinear, "fern", "fern",
                                                    sparse=True)

HingeTreeFusion = _fusion_function("HingeTreeFusion", "tree", "tree")
HingeFernFusion = _fusion_function("HingeFernFusion", "fern", "fern")
HingeTreeFusionFusedLinear = _fusion_fused_linear_function("HingeTreeFusionFusedLinear", HingeTreeFusion, "tree", "tree")
HingeFernFusionFusedLinear = _fusion_fused_linear_function("HingeFernFusionFusedLinear", HingeFernFusion, "fern", "fern")

HingeTreeConv1d = _conv_function("HingeTreeConv1d", "tree", 1, "tree")
HingeTreeConv2d = _conv_function("HingeTreeConv2d", "tree", 2, "tree")
HingeTreeConv3d = _conv_function("HingeTreeConv3d", "tree", 3, "tree")
HingeFernConv1d = _conv_function("HingeFernConv1d", "fern", 1, "fern")
HingeFernConv2d = _conv_function("HingeFernConv2d", "fern", 2, "fern")
HingeFernConv3d = _conv_function("HingeFernConv3d", "fern", 3, "fern")


class HingeTrie(torch.autograd.Function):
    @staticmethod
    def forward(ctx, inData, inThresholds, inOrdinals, inWeights):
        ctx.save_for_backward(inData, inThresholds, inOrdinals, inWeights)
        return hingetree_cpp.trie_forward(inData, inThresholds, inOrdinals, inWeights)

    @staticmethod
    def backward(ctx, outDataGrad):
        _refuse_deterministic(outDataGrad, "backpropagation of hinge trie")
        return tuple(hingetree_cpp.trie_backward(*_interleave(ctx.saved_tensors, ctx.needs_input_grad),
                                                 outDataGrad.contiguous()))

    @staticmethod
    def init_medians(inData, inThresholds, inOrdinals, inWeights):
        return hingetree_cpp.trie_init_medians(inData, inThresholds, inOrdinals, inWeights)
