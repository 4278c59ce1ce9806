"""numpy front end of the C restatement in hinge_oracle.c (test infrastructure only).

Only tests, the smoke check and the CPU-baseline legs of the benchmark import this module.
The product path never does: it has no CPU fallback.

All arrays are C-contiguous; x is float32 [B, C, *inner], thr float32 [T, N], ord int64 [T, N],
w float32 [T, L, *extra].  ``kind`` is "tree" or "fern".
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = [os.path.join(HERE, name) for name in ("hinge_oracle.c", "hinge_oracle_conv.c", "hinge_oracle_trie.c")]
LIB = os.path.join(HERE, "libhinge_oracle.so")

_KIND = {"tree": 0, "fern": 1}
_lib = None


def build(force=False):
    """Compile the C sources with gcc (no FMA contraction, like the reference's x86-64 -O2 build)."""
    inputs = SOURCES + [os.path.join(HERE, "hinge_oracle_terms.h")]
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < max(os.path.getmtime(s) for s in inputs):
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c11",
                        "-o", LIB] + SOURCES + ["-lm"], check=True)
    return LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _dims(x, w):
    B, C = x.shape[0], x.shape[1]
    K = int(np.prod(x.shape[2:], dtype=np.int64))
    T, L = w.shape[0], w.shape[1]
    M = int(np.prod(w.shape[2:], dtype=np.int64))
    return B, C, K, T, L, M


def _i(v):
    return ctypes.c_int64(int(v))


def forward(kind, x, thr, ord_, w, vec=None):
    x, thr, ord_, w = _f32(x), _f32(thr), _i64(ord_), _f32(w)
    vec = None if vec is None else _f32(vec)
    B, C, K, T, L, M = _dims(x, w)
    out = np.empty((B, T) + x.shape[2:] + w.shape[2:], dtype=np.float32)
    rc = lib().ho_forward(_KIND[kind], _p(x), _p(vec), _i(0 if vec is None else vec.shape[1]), _p(thr), _p(ord_),
                          _p(w), _p(out), _i(B), _i(C), _i(K), _i(T), _i(L), _i(M))
    if rc != 0:
        raise ValueError("leaf count is not a power of two")
    return out


def maps(kind, x, thr, ord_, w):
    """Returns (leafmap int64, margins float32, margin ordinals int64, reachability int64 [T, L])."""
    x, thr, ord_ = _f32(x), _f32(thr), _i64(ord_)
    B, C, K, T, L, _ = _dims(x, w)
    shape = (B, T) + x.shape[2:]
    leaf = np.empty(shape, dtype=np.int64)
    margin = np.empty(shape, dtype=np.float32)
    mord = np.empty(shape, dtype=np.int64)
    reach = np.empty((T, L), dtype=np.int64)
    rc = lib().ho_maps(_KIND[kind], _p(x), _p(thr), _p(ord_), _p(leaf), _p(margin), _p(mord), _p(reach),
                       _i(B), _i(C), _i(K), _i(T), _i(L))
    if rc != 0:
        raise ValueError("leaf count is not a power of two")
    return leaf, margin, mord, reach


def backward(kind, x, thr, ord_, w, g, vec=None, need=(True, True, True)):
    """Returns (gx, gthr, gw) or, with vec given, (gimg, gvec, gthr, gw); entries not needed are None."""
    x, thr, ord_, w, g = _f32(x), _f32(thr), _i64(ord_), _f32(w), _f32(g)
    vec = None if vec is None else _f32(vec)
    B, C, K, T, L, M = _dims(x, w)
    gx = np.zeros_like(x) if need[0] else None
    gvec = np.zeros_like(vec) if (need[0] and vec is not None) else None
    gthr = np.zeros_like(thr) if need[1] else None
    gw = np.zeros_like(w) if need[2] else None
    rc = lib().ho_backward(_KIND[kind], _p(x), _p(vec), _i(0 if vec is None else vec.shape[1]), _p(thr), _p(ord_),
                           _p(w), _p(g), _p(gx), _p(gvec), _p(gthr), _p(gw),
                           _i(B), _i(C), _i(K), _i(T), _i(L), _i(M))
    if rc != 0:
        raise ValueError("leaf count is not a power of two")
    if vec is None:
        return gx, gthr, gw
    return gx, gvec, gthr, gw


def backward_magnitudes(kind, x, thr, ord_, w, g):
    """Sum of |term| added into each element of (gx, gthr, gw), float64: the scale of a tolerance."""
    x, thr, ord_, w, g = _f32(x), _f32(thr), _i64(ord_), _f32(w), _f32(g)
    B, C, K, T, L, M = _dims(x, w)
    ax, athr, aw = np.zeros(x.shape), np.zeros(thr.shape), np.zeros(w.shape)
    rc = lib().ho_backward_magnitudes(_KIND[kind], _p(x), _p(thr), _p(ord_), _p(w), _p(g), _p(ax), _p(athr), _p(aw),
                                      _i(B), _i(C), _i(K), _i(T), _i(L), _i(M))
    if rc != 0:
        raise ValueError("leaf count is not a power of two")
    return ax, athr, aw


def magnitudes(backward_fn, *args, **kwargs):
    """Runs one of this module's backward functions (backward, linear_backward, conv_backward,
    trie_backward) with every term replaced by its absolute value: the result has, per gradient
    element, the sum of |term| over all contributions (float32), which is what a relative
    tolerance of a sum computed in another order has to be multiplied with."""
    lib().ho_set_magnitude_mode(1)
    try:
        return backward_fn(*args, **kwargs)
    finally:
        lib().ho_set_magnitude_mode(0)


def linear_forward(kind, x, thr, ord_, w, lin, bias, vec=None):
    """Trees followed by the linear layer over the tree dimension: out [B, O, *inner, *extra]."""
    x, thr, ord_, w, lin, bias = _f32(x), _f32(thr), _i64(ord_), _f32(w), _f32(lin), _f32(bias)
    vec = None if vec is None else _f32(vec)
    B, C, K, T, L, M = _dims(x, w)
    O = lin.shape[0]
    out = np.empty((B, O) + x.shape[2:] + w.shape[2:], dtype=np.float32)
    rc = lib().ho_linear_forward(_KIND[kind], _p(x), _p(vec), _i(0 if vec is None else vec.shape[1]), _p(thr),
                                 _p(ord_), _p(w), _p(lin), _p(bias), _p(out), _i(B), _i(C), _i(K), _i(T), _i(L), _i(M),
                                 _i(O))
    if rc != 0:
        raise ValueError("leaf count is not a power of two")
    return out


def linear_backward(kind, x, thr, ord_, w, lin, g, vec=None):
    """Returns (gx, [gvec,] gthr, gw, glin, gbias)."""
    x, thr, ord_, w, lin, g = _f32(x), _f32(thr), _i64(ord_), _f32(w), _f32(lin), _f32(g)
    vec = None if vec is None else _f32(vec)
    B, C, K, T, L, M = _dims(x, w)
    O = lin.shape[0]
    gx, gthr, gw, glin = np.zeros_like(x), np.zeros_like(thr), np.zeros_like(w), np.zeros_like(lin)
    gvec = None if vec is None else np.zeros_like(vec)
    gbias = np.zeros(O, dtype=np.float32)
    rc = lib().ho_linear_backward(_KIND[kind], _p(x), _p(vec), _i(0 if vec is None else vec.shape[1]), _p(thr),
                                  _p(ord_), _p(w), _p(lin), _p(g), _p(gx), _p(gvec), _p(gthr), _p(gw), _p(glin),
                                  _p(gbias), _i(B), _i(C), _i(K), _i(T), _i(L), _i(M), _i(O))
    if rc != 0:
        raise ValueError("leaf count is not a power of two")
    if vec is None:
        return gx, gthr, gw, glin, gbias
    return gx, gvec, gthr, gw, glin, gbias


def trie_forward(x, thr, ord_, w):
    """Hinge trie: w is [T, 2^depth - 1, *extra] (one row per internal vertex)."""
    x, thr, ord_, w = _f32(x), _f32(thr), _i64(ord_), _f32(w)
    B, C, K, T, N, M = _dims(x, w)
    out = np.empty((B, T) + x.shape[2:] + w.shape[2:], dtype=np.float32)
    if lib().ho_trie_forward(_p(x), _p(thr), _p(ord_), _p(w), _p(out), _i(B), _i(C), _i(K), _i(T), _i(N), _i(M)) != 0:
        raise ValueError("threshold count + 1 is not a power of two")
    return out


def trie_backward(x, thr, ord_, w, g):
    x, thr, ord_, w, g = _f32(x), _f32(thr), _i64(ord_), _f32(w), _f32(g)
    B, C, K, T, N, M = _dims(x, w)
    gx, gthr, gw = np.zeros_like(x), np.zeros_like(thr), np.zeros_like(w)
    if lib().ho_trie_backward(_p(x), _p(thr), _p(ord_), _p(w), _p(g), _p(gx), _p(gthr), _p(gw), _i(B), _i(C), _i(K),
                              _i(T), _i(N), _i(M)) != 0:
        raise ValueError("threshold count + 1 is not a power of two")
    return gx, gthr, gw


def _i64s(values):
    arr = (ctypes.c_int64 * len(values))(*[int(v) for v in values])
    return arr


def _geometry(x, kernel, stride, padding, dilation):
    dims = x.ndim - 2
    return dims, _i64s(x.shape[2:]), _i64s(kernel), _i64s(stride), _i64s(padding), _i64s(dilation)


def conv_output_size(size, kernel, stride, padding, dilation):
    dims = len(size)
    osize = (ctypes.c_int64 * dims)()
    count = lib().ho_conv_output_size(dims, _i64s(size), _i64s(kernel), _i64s(stride), _i64s(padding), _i64s(dilation),
                                      osize)
    if count < 0:
        raise ValueError("bad convolution geometry")
    return tuple(osize)


def conv_forward(kind, x, thr, ord_, w, kernel, stride, padding, dilation):
    """x [B, Ci, *size]; thr, ord [Co, Ci, N]; w [Co, Ci, L, *extra] -> out [B, Co, *osize, *extra]."""
    x, thr, ord_, w = _f32(x), _f32(thr), _i64(ord_), _f32(w)
    dims, size, kernel_, stride_, pad_, dil_ = _geometry(x, kernel, stride, padding, dilation)
    osize = conv_output_size(x.shape[2:], kernel, stride, padding, dilation)
    B, Ci, Co, L = x.shape[0], x.shape[1], w.shape[0], w.shape[2]
    M = int(np.prod(w.shape[3:], dtype=np.int64))
    out = np.empty((B, Co) + osize + w.shape[3:], dtype=np.float32)
    rc = lib().ho_conv_forward(_KIND[kind], dims, _p(x), _p(thr), _p(ord_), _p(w), _p(out), _i(B), _i(Ci), _i(Co), _i(L),
                               _i(M), size, kernel_, stride_, pad_, dil_)
    if rc != 0:
        raise ValueError("bad convolution arguments")
    return out


def conv_backward(kind, x, thr, ord_, w, g, kernel, stride, padding, dilation):
    x, thr, ord_, w, g = _f32(x), _f32(thr), _i64(ord_), _f32(w), _f32(g)
    dims, size, kernel_, stride_, pad_, dil_ = _geometry(x, kernel, stride, padding, dilation)
    B, Ci, Co, L = x.shape[0], x.shape[1], w.shape[0], w.shape[2]
    M = int(np.prod(w.shape[3:], dtype=np.int64))
    gx, gthr, gw = np.zeros_like(x), np.zeros_like(thr), np.zeros_like(w)
    rc = lib().ho_conv_backward(_KIND[kind], dims, _p(x), _p(thr), _p(ord_), _p(w), _p(g), _p(gx), _p(gthr), _p(gw),
                                _i(B), _i(Ci), _i(Co), _i(L), _i(M), size, kernel_, stride_, pad_, dil_)
    if rc != 0:
        raise ValueError("bad convolution arguments")
    return gx, gthr, gw


def contract(x, window, padding):
    """[B, C, *size] -> [B, C, *osize, *window] (non-overlapping windows, zero padded)."""
    x = np.ascontiguousarray(x)
    dims = x.ndim - 2
    osize = tuple((s + 2 * p - w_) // w_ + 1 for s, p, w_ in zip(x.shape[2:], padding, window))
    out = np.empty(x.shape[:2] + osize + tuple(window), dtype=x.dtype)
    rc = lib().ho_contract(dims, x.dtype.itemsize, _p(x), _p(out), _i(x.shape[0] * x.shape[1]), _i64s(x.shape[2:]),
                           _i64s(window), _i64s(padding))
    if rc != 0:
        raise ValueError("bad contract arguments")
    return out


def expand(x, padding):
    """[B, C, *osize, *window] -> [B, C, *size]: the inverse of contract."""
    x = np.ascontiguousarray(x)
    dims = (x.ndim - 2) // 2
    osize, window = x.shape[2:2 + dims], x.shape[2 + dims:]
    size = (ctypes.c_int64 * dims)()
    if lib().ho_expand(dims, x.dtype.itemsize, _p(x), None, _i(0), _i64s(osize), _i64s(window), _i64s(padding), size) != 0:
        raise ValueError("bad expand arguments")
    out = np.empty(x.shape[:2] + tuple(size), dtype=x.dtype)
    rc = lib().ho_expand(dims, x.dtype.itemsize, _p(x), _p(out), _i(x.shape[0] * x.shape[1]), _i64s(osize), _i64s(window),
                         _i64s(padding), size)
    if rc != 0:
        raise ValueError("bad expand arguments")
    return out
