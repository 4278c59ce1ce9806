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
SRC = os.path.join(HERE, "hinge_oracle.c")
LIB = os.path.join(HERE, "libhinge_oracle.so")

_KIND = {"tree": 0, "fern": 1}
_lib = None


def build(force=False):
    """Compile hinge_oracle.c with gcc (no FMA contraction, like the reference's x86-64 -O2 build)."""
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
        subprocess.run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-std=c11",
                        "-o", LIB, SRC, "-lm"], check=True)
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
