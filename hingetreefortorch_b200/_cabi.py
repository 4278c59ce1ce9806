"""ctypes binding of the C ABI in include/hingetree_b200.h.

This is the thinnest possible caller of the library: it passes raw device pointers of torch
tensors and the current CUDA stream.  The parity tests and the benchmark go through it so
that they exercise exactly the symbols a foreign binding would.  torch is used for device
memory and streams only.
"""
import ctypes
import os

from . import _build

HT_KIND = {"tree": 0, "fern": 1}
HT_DETERMINISTIC = 1
HT_WORKSPACE_FOR_BACKWARD = 2
HT_SAVE_FOR_BACKWARD = 4
HT_SAVED_FORWARD = 8
HT_FLAG_ORDINAL_RANGE = 1
HT_FLAG_PIPELINE_TIMEOUT = 0x80000000  # a bounded wait inside a kernel ran out: outputs incomplete

# every symbol include/hingetree_b200.h declares (checked by the CPU test-suite)
SYMBOLS = [
    "ht_version", "ht_status_string", "ht_last_cuda_error", "ht_forest_workspace_bytes", "ht_forest_forward_saves", "ht_launch_count", "ht_selftest_bounded_wait",
    "ht_forest_forward_f32", "ht_forest_leafmap_f32", "ht_forest_marginmap_f32",
    "ht_forest_reachability_f32", "ht_forest_backward_f32",
    "ht_forest_forward_f64", "ht_forest_leafmap_f64", "ht_forest_marginmap_f64", "ht_forest_reachability_f64",
    "ht_forest_backward_f64",
    "ht_forest_static_scratch_bytes", "ht_forest_forward_static_f32",
    "ht_forest_fusion_workspace_bytes", "ht_forest_fusion_forward_f32", "ht_forest_fusion_backward_f32",
    "ht_forest_linear_workspace_bytes", "ht_forest_linear_forward_f32", "ht_forest_linear_backward_f32",
    "ht_conv_output_size", "ht_conv_workspace_bytes", "ht_conv_forward_f32", "ht_conv_backward_f32",
    "ht_contract", "ht_expand",
    "ht_trie_forward_f32", "ht_trie_backward_f32", "ht_forest_touched_f32", "ht_linear_tf32_stats_f32",
    "ht_forest_linear_workspace_bytes_f64", "ht_forest_fusion_forward_f64", "ht_forest_fusion_backward_f64",
    "ht_forest_linear_forward_f64", "ht_forest_linear_backward_f64", "ht_conv_forward_f64", "ht_conv_backward_f64",
    "ht_trie_forward_f64", "ht_trie_backward_f64", "ht_forest_touched_f64",
    "ht_forest_normalised_workspace_bytes", "ht_forest_normalised_forward_f32", "ht_forest_normalised_backward_f32",
    "ht_batchnorm_input_grad_f32", "ht_batchnorm_statistics_f32",
    "ht_init_medians_workspace_bytes", "ht_init_medians_f32", "ht_init_medians_f64", "ht_thresholds_f32", "ht_thresholds_f64",
]


class ConvProblem(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("depth", ctypes.c_int32), ("dims", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("B", ctypes.c_int64), ("Ci", ctypes.c_int64), ("Co", ctypes.c_int64),
                ("M", ctypes.c_int64), ("size", ctypes.c_int64 * 3), ("kernel", ctypes.c_int64 * 3),
                ("stride", ctypes.c_int64 * 3), ("padding", ctypes.c_int64 * 3), ("dilation", ctypes.c_int64 * 3)]


def _triple(values, fill):
    values = list(values) + [fill] * (3 - len(values))
    return (ctypes.c_int64 * 3)(*values)


class Conv:
    """Convolutional hinge trees through the C ABI: x [B,Ci,*size], thr/ord [Co,Ci,N], w [Co,Ci,L,*extra]."""

    def __init__(self, kind, x, w, kernel, stride, padding, dilation):
        import math
        import torch
        dims = x.dim() - 2
        L = w.shape[2]
        self.problem = ConvProblem(HT_KIND[kind], L.bit_length() - 1, dims, 0, x.shape[0], x.shape[1], w.shape[0],
                                   math.prod(w.shape[3:]), _triple(x.shape[2:], 1), _triple(kernel, 1),
                                   _triple(stride, 1), _triple(padding, 0), _triple(dilation, 1))
        lib = library()
        lib.ht_conv_workspace_bytes.restype = ctypes.c_size_t
        osize = (ctypes.c_int64 * 3)()
        _check(lib.ht_conv_output_size(ctypes.byref(self.problem), osize))
        self.out_shape = (x.shape[0], w.shape[0]) + tuple(osize[:dims]) + tuple(w.shape[3:])
        nbytes = lib.ht_conv_workspace_bytes(ctypes.byref(self.problem))
        self.workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=x.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=x.device)

    def _tail(self, x):
        return (_ptr(self.workspace), ctypes.c_size_t(self.workspace.numel()), _ptr(self.status), _stream(x))

    def forward(self, x, thr, ord_, w):
        import torch
        out = torch.empty(self.out_shape, dtype=torch.float32, device=x.device)
        _check(library().ht_conv_forward_f32(ctypes.byref(self.problem), _ptr(x), _ptr(thr), _ptr(ord_), _ptr(w),
                                             _ptr(out), *self._tail(x)))
        return out

    def backward(self, x, thr, ord_, w, g):
        import torch
        outs = [torch.empty_like(t) for t in (x, thr, w)]
        _check(library().ht_conv_backward_f32(ctypes.byref(self.problem), _ptr(x), _ptr(thr), _ptr(ord_), _ptr(w),
                                              _ptr(g), *[_ptr(t) for t in outs], *self._tail(x)))
        return outs


def _i64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(v) for v in values])


def contract(x, window, padding):
    import torch
    dims = len(window)
    osize = [(s + 2 * p - w) // w + 1 for s, p, w in zip(x.shape[2:], padding, window)]
    out = torch.empty(tuple(x.shape[:2]) + tuple(osize) + tuple(window), dtype=x.dtype, device=x.device)
    _check(library().ht_contract(dims, x.element_size(), _ptr(x), _ptr(out), ctypes.c_int64(x.shape[0] * x.shape[1]),
                                 _i64_array(x.shape[2:]), _i64_array(window), _i64_array(padding), _stream(x)))
    return out


def expand(x, padding):
    import torch
    dims = len(padding)
    osize, window = x.shape[2:2 + dims], x.shape[2 + dims:]
    size = [o * w - ((2 * p) // w) * w for o, w, p in zip(osize, window, padding)]
    out = torch.empty(tuple(x.shape[:2]) + tuple(size), dtype=x.dtype, device=x.device)
    _check(library().ht_expand(dims, x.element_size(), _ptr(x), _ptr(out), ctypes.c_int64(x.shape[0] * x.shape[1]),
                               _i64_array(osize), _i64_array(window), _i64_array(padding), _stream(x)))
    return out


class ForestProblem(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("depth", ctypes.c_int32), ("B", ctypes.c_int64), ("C", ctypes.c_int64),
                ("K", ctypes.c_int64), ("T", ctypes.c_int64), ("M", ctypes.c_int64), ("flags", ctypes.c_uint32),
                ("reserved", ctypes.c_uint32)]


class HingeTreeError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("hingetree_b200 status %d: %s" % (status, message))
        self.status = status


_lib = None


def library():
    """Load libhingetree_b200.so from the source tree.  Fails loudly when it was not built."""
    global _lib
    if _lib is None:
        path = _build.library_path()
        if not os.path.exists(path):
            raise ImportError("%s is missing: build it with `python -m hingetreefortorch_b200._build` "
                              "(there is no fallback path)" % path)
        lib = ctypes.CDLL(path)
        lib.ht_status_string.restype = ctypes.c_char_p
        lib.ht_status_string.argtypes = [ctypes.c_int]
        lib.ht_forest_workspace_bytes.restype = ctypes.c_size_t
        lib.ht_forest_workspace_bytes.argtypes = [ctypes.POINTER(ForestProblem)]
        lib.ht_forest_static_scratch_bytes.restype = ctypes.c_size_t
        lib.ht_launch_count.restype = ctypes.c_uint64
        _lib = lib
    return _lib


def _check(rc):
    if rc != 0:
        raise HingeTreeError(rc, library().ht_status_string(rc).decode())


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(t):
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def forest_problem(kind, x, w, deterministic=False):
    import math
    L = w.shape[1]
    depth = L.bit_length() - 1
    if L <= 0 or (1 << depth) != L:
        raise ValueError("leaf count %d is not a power of two" % L)
    return ForestProblem(HT_KIND[kind], depth, x.shape[0], x.shape[1], math.prod(x.shape[2:]), w.shape[0],
                         math.prod(w.shape[2:]), HT_DETERMINISTIC if deterministic else 0, 0)


class Forest:
    """Scratch memory and status word for repeated calls on one problem shape."""

    def __init__(self, kind, x, w, deterministic=False, backward_workspace=True):
        import torch
        self.kind = kind
        self.problem = forest_problem(kind, x, w, deterministic)
        self.problem.flags |= HT_WORKSPACE_FOR_BACKWARD if backward_workspace else 0
        nbytes = library().ht_forest_workspace_bytes(ctypes.byref(self.problem))
        self.workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=x.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=x.device)
        self.out_shape = tuple(x.shape[:1]) + tuple(w.shape[:1]) + tuple(x.shape[2:]) + tuple(w.shape[2:])
        self.map_shape = tuple(x.shape[:1]) + tuple(w.shape[:1]) + tuple(x.shape[2:])

    def _tail(self, x):
        return (_ptr(self.workspace), ctypes.c_size_t(self.workspace.numel()), _ptr(self.status), _stream(x))

    def _with_flags(self, extra):
        problem = ForestProblem.from_buffer_copy(self.problem)
        problem.flags |= extra
        return problem

    def saves_forward(self):
        """Whether forward(save=True) keeps the traversal for backward(saved=True) on this problem."""
        return bool(library().ht_forest_forward_saves(ctypes.byref(self.problem)))

    def forward(self, x, thr, ord_, w, out=None, save=False):
        import torch
        if out is None:
            out = torch.empty(self.out_shape, dtype=torch.float32, device=x.device)
        problem = self._with_flags(HT_SAVE_FOR_BACKWARD) if save else self.problem
        _check(library().ht_forest_forward_f32(ctypes.byref(problem), _ptr(x), _ptr(thr), _ptr(ord_), _ptr(w),
                                               _ptr(out), *self._tail(x)))
        return out

    def forward_static(self, x, thr, ord_, w, out=None):
        """The forward through the entry point that uses the library's built-in scratch array."""
        import torch
        if out is None:
            out = torch.empty(self.out_shape, dtype=torch.float32, device=x.device)
        _check(library().ht_forest_forward_static_f32(ctypes.byref(self.problem), _ptr(x), _ptr(thr), _ptr(ord_),
                                                      _ptr(w), _ptr(out), _ptr(self.status), _stream(x)))
        return out

    def leafmap(self, x, thr, ord_):
        import torch
        leaf = torch.empty(self.map_shape, dtype=torch.int64, device=x.device)
        _check(library().ht_forest_leafmap_f32(ctypes.byref(self.problem), _ptr(x), _ptr(thr), _ptr(ord_), _ptr(leaf),
                                               *self._tail(x)))
        return leaf

    def marginmap(self, x, thr, ord_):
        import torch
        margin = torch.empty(self.map_shape, dtype=torch.float32, device=x.device)
        mord = torch.empty(self.map_shape, dtype=torch.int64, device=x.device)
        _check(library().ht_forest_marginmap_f32(ctypes.byref(self.problem), _ptr(x), _ptr(thr), _ptr(ord_),
                                                 _ptr(margin), _ptr(mord), *self._tail(x)))
        return margin, mord

    def reachability(self, x, thr, ord_):
        import torch
        counts = torch.empty((self.problem.T, 1 << self.problem.depth), dtype=torch.int64, device=x.device)
        _check(library().ht_forest_reachability_f32(ctypes.byref(self.problem), _ptr(x), _ptr(thr), _ptr(ord_),
                                                    _ptr(counts), *self._tail(x)))
        return counts

    def backward(self, x, thr, ord_, w, g, need=(True, True, True), outs=None, saved=False):
        """saved=True: the last call on this object was forward(save=True) on the same tensors."""
        import torch
        if outs is None:  # NaN-filled: an element the library fails to write shows in every comparison
            outs = (torch.full_like(x, float("nan")) if need[0] else None, torch.full_like(thr, float("nan")) if need[1] else None,
                    torch.full_like(w, float("nan")) if need[2] else None)
        problem = self._with_flags(HT_SAVED_FORWARD) if saved else self.problem
        _check(library().ht_forest_backward_f32(ctypes.byref(problem), _ptr(x), _ptr(thr), _ptr(ord_), _ptr(w),
                                                _ptr(g), _ptr(outs[0]), _ptr(outs[1]), _ptr(outs[2]), *self._tail(x)))
        return outs

    def ordinal_flags(self):
        """Reads the device status word (blocks until the stream has drained); raises when a kernel gave up on
        a bounded wait, returns the other flag bits (HT_FLAG_ORDINAL_RANGE)."""
        flags = int(self.status.item()) & 0xffffffff
        if flags & HT_FLAG_PIPELINE_TIMEOUT:
            raise HingeTreeError(-3, "a bounded wait inside a kernel ran out; outputs are incomplete")
        return flags


class ForestFamily:
    """Fusion (image + vector) and fused-linear calls on one problem shape; vec / lin are optional."""

    def __init__(self, kind, x, w, vec=None, lin=None):
        import torch
        self.problem = forest_problem(kind, x, w)
        self.vec_channels = 0 if vec is None else vec.shape[1]
        self.out_channels = 0 if lin is None else lin.shape[0]
        lib = library()
        lib.ht_forest_linear_workspace_bytes.restype = ctypes.c_size_t
        lib.ht_forest_fusion_workspace_bytes.restype = ctypes.c_size_t
        nbytes = max(lib.ht_forest_linear_workspace_bytes(ctypes.byref(self.problem)),
                     lib.ht_forest_fusion_workspace_bytes(ctypes.byref(self.problem)))
        self.workspace = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=x.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=x.device)
        inner = tuple(x.shape[2:]) + tuple(w.shape[2:])
        self.out_shape = (x.shape[0], w.shape[0] if lin is None else lin.shape[0]) + inner

    def _tail(self, x):
        return (_ptr(self.workspace), ctypes.c_size_t(self.workspace.numel()), _ptr(self.status), _stream(x))

    def fusion_forward(self, img, vec, thr, ord_, w):
        import torch
        out = torch.empty(self.out_shape, dtype=torch.float32, device=img.device)
        _check(library().ht_forest_fusion_forward_f32(ctypes.byref(self.problem), _ptr(img), _ptr(vec),
                                                      ctypes.c_int64(self.vec_channels), _ptr(thr), _ptr(ord_), _ptr(w),
                                                      _ptr(out), *self._tail(img)))
        return out

    def fusion_backward(self, img, vec, thr, ord_, w, g):
        import torch
        outs = [torch.empty_like(t) for t in (img, vec, thr, w)]
        _check(library().ht_forest_fusion_backward_f32(ctypes.byref(self.problem), _ptr(img), _ptr(vec),
                                                       ctypes.c_int64(self.vec_channels), _ptr(thr), _ptr(ord_), _ptr(w),
                                                       _ptr(g), *[_ptr(t) for t in outs], *self._tail(img)))
        return outs

    def linear_forward(self, x, vec, thr, ord_, w, lin, bias):
        import torch
        out = torch.empty(self.out_shape, dtype=torch.float32, device=x.device)
        _check(library().ht_forest_linear_forward_f32(ctypes.byref(self.problem), ctypes.c_int64(self.out_channels),
                                                      _ptr(x), _ptr(vec), ctypes.c_int64(self.vec_channels), _ptr(thr),
                                                      _ptr(ord_), _ptr(w), _ptr(lin), _ptr(bias), _ptr(out),
                                                      *self._tail(x)))
        return out

    def linear_backward(self, x, vec, thr, ord_, w, lin, g):
        """Returns (gx, gvec or None, gthr, gw, glin)."""
        import torch
        gx, gthr, gw, glin = [torch.empty_like(t) for t in (x, thr, w, lin)]
        gvec = None if vec is None else torch.empty_like(vec)
        _check(library().ht_forest_linear_backward_f32(ctypes.byref(self.problem), ctypes.c_int64(self.out_channels),
                                                       _ptr(x), _ptr(vec), ctypes.c_int64(self.vec_channels), _ptr(thr),
                                                       _ptr(ord_), _ptr(w), _ptr(lin), _ptr(g), _ptr(gx), _ptr(gvec),
                                                       _ptr(gthr), _ptr(gw), _ptr(glin), *self._tail(x)))
        return gx, gvec, gthr, gw, glin


def linear_tf32_stats(x, w, status=None):
    """z = x @ w.T on the tensor cores (TF32 products, fp32 accumulation) with the column sums and sums of
    squares of z: returns (z [M, N], colsum [N], colsumsq [N])."""
    import torch
    M, K = x.shape
    N = w.shape[0]
    z = torch.empty((M, N), dtype=torch.float32, device=x.device)
    colsum = torch.empty(N, dtype=torch.float32, device=x.device)
    colsumsq = torch.empty(N, dtype=torch.float32, device=x.device)
    _check(library().ht_linear_tf32_stats_f32(_ptr(x), _ptr(w), _ptr(z), _ptr(colsum), _ptr(colsumsq), ctypes.c_int64(M),
                                              ctypes.c_int64(N), ctypes.c_int64(K), _ptr(status), _stream(x)))
    return z, colsum, colsumsq


def selftest_bounded_wait(status):
    """Runs the library's self test of a bounded wait (a one-warp kernel waits a few tries on a barrier that
    nothing arrives on): afterwards the int32 status word holds HT_FLAG_PIPELINE_TIMEOUT."""
    _check(library().ht_selftest_bounded_wait(_ptr(status), _stream(status)))


def init_medians(kind, x, thr, ord_):
    """Median initialisation of the thresholds on the device (thr is overwritten): x [B, C, *inner], thr and
    ord_ [T, N] on the same CUDA device, float32 or float64."""
    import torch
    lib = library()
    lib.ht_init_medians_workspace_bytes.restype = ctypes.c_size_t
    B, C = x.shape[0], x.shape[1]
    K = 1
    for d in x.shape[2:]:
        K *= d
    T, N = thr.shape
    depth = N if kind == "fern" else (N + 1).bit_length() - 1
    code = {"tree": 0, "fern": 1}[kind]
    need = lib.ht_init_medians_workspace_bytes(code, ctypes.c_int64(B), ctypes.c_int64(K), ctypes.c_int64(T), depth,
                                               x.element_size())
    ws = torch.empty(max(int(need), 1), dtype=torch.uint8, device=x.device)
    fn = lib.ht_init_medians_f64 if x.dtype == torch.float64 else lib.ht_init_medians_f32
    _check(fn(code, _ptr(x), _ptr(thr), _ptr(ord_), ctypes.c_int64(B), ctypes.c_int64(C), ctypes.c_int64(K),
              ctypes.c_int64(T), depth, _ptr(ws), ctypes.c_size_t(ws.numel()), _stream(x)))
    return thr


def thresholds(fix, thr, ord_):
    """check (fix False: 1 per consistent tree) or fix (1 per changed tree; thr is edited) on the device."""
    import torch
    T, N = thr.shape
    depth = (N + 1).bit_length() - 1
    result = torch.zeros(T, dtype=torch.uint8, device=thr.device)
    fn = library().ht_thresholds_f64 if thr.dtype == torch.float64 else library().ht_thresholds_f32
    _check(fn(1 if fix else 0, _ptr(thr), _ptr(ord_), ctypes.c_int64(T), depth, _ptr(result), _stream(thr)))
    return result
