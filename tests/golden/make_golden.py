"""Generates the golden vectors in this directory by running the UNMODIFIED reference.

The reference CPU implementation is compiled by oracle/build_ref.py (from the reference
checkout, into oracle/_ref/) and called here on small seeded inputs; inputs and outputs are
stored as .npz files.  The reference cannot travel to a GPU machine, the vectors can.

    python oracle/build_ref.py && python tests/golden/make_golden.py

Cases cover trees and ferns, tabular and image-shaped inputs, scalar and multi-dimensional
leaf outputs, and adversarial values: exact ties in |margin|, margins that are exactly zero,
infinities, duplicated features along a path.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402


def decisions(kind, depth):
    return depth if kind == "fern" else 2 ** depth - 1


def make_case(seed, kind, B, C, inner, T, depth, extra, adversarial=False):
    gen = torch.Generator().manual_seed(seed)
    N = decisions(kind, depth)
    x = torch.randn((B, C) + tuple(inner), generator=gen)
    thr = torch.rand((T, N), generator=gen) * 6 - 3
    ord_ = torch.randint(0, C, (T, N), generator=gen)
    w = torch.randn((T, 2 ** depth) + tuple(extra), generator=gen)
    if adversarial:
        # quantise so that exact ties and exact zeros occur, and plant special values
        x = torch.round(x * 2) / 2
        thr = torch.round(thr * 2) / 2
        flat = x.view(-1)
        flat[0] = float("inf")
        flat[1] = float("-inf")
        flat[2] = 1e-42  # denormal
        ord_[:, : min(N, 3)] = ord_[:, :1]  # the same feature repeated along the path
    return x, thr, ord_, w, gen


def forest_cases():
    cases = []
    seed = 100
    for kind in ("tree", "fern"):
        for (B, C, inner, T, depth, extra, adv) in [
            (5, 7, (), 3, 1, (), False),
            (9, 11, (), 6, 3, (), False),
            (4, 5, (3,), 5, 4, (2,), False),
            (3, 6, (2, 3), 4, 2, (2, 2), False),
            (33, 16, (), 9, 5, (3,), False),
            (16, 4, (), 7, 3, (), True),
            (6, 3, (5,), 4, 3, (2,), True),
        ]:
            seed += 1
            cases.append((seed, kind, B, C, inner, T, depth, extra, adv))
    return cases


def main():
    ref = build_ref.load()
    out = {}
    for idx, (seed, kind, B, C, inner, T, depth, extra, adv) in enumerate(forest_cases()):
        x, thr, ord_, w, gen = make_case(seed, kind, B, C, inner, T, depth, extra, adv)
        f = getattr(ref, kind + "_forward")(x, thr, ord_, w)
        g = torch.randn(f.shape, generator=gen)
        gx, gthr, _, gw = getattr(ref, kind + "_backward")(x, True, thr, True, ord_, False, w, True, g)
        leaf = getattr(ref, kind + "_leafmap")(x, thr, ord_, w)
        margin, mord = getattr(ref, kind + "_marginmap")(x, thr, ord_, w)
        reach = getattr(ref, kind + "_reachability")(x, thr, ord_, w)
        p = "forest%02d_" % idx
        out[p + "kind"] = np.array(kind)
        for name, t in [("x", x), ("thr", thr), ("ord", ord_), ("w", w), ("g", g), ("out", f), ("gx", gx),
                        ("gthr", gthr), ("gw", gw), ("margin", margin), ("margin_ord", mord)]:
            out[p + name] = t.numpy()
        # the reference CPU path returns these two as floats; they hold exact small integers
        out[p + "leaf"] = leaf.numpy().astype(np.int64)
        out[p + "reach"] = reach.numpy().astype(np.int64)
    out["forest_count"] = np.array(len(forest_cases()))

    # threshold hygiene: before / after fix_thresholds, and the check verdicts
    gen = torch.Generator().manual_seed(7)
    thr = torch.rand((12, 31), generator=gen) * 6 - 3
    ord_ = torch.randint(0, 3, (12, 31), generator=gen)
    w = torch.randn((12, 32), generator=gen)
    out["hygiene_thr_before"] = thr.numpy().copy()
    out["hygiene_ord"] = ord_.numpy()
    out["hygiene_check_before"] = np.array(ref.tree_check_thresholds(thr, ord_, w))
    out["hygiene_changed"] = np.array(ref.tree_fix_thresholds(thr, ord_, w))
    out["hygiene_thr_after"] = thr.numpy().copy()
    out["hygiene_check_after"] = np.array(ref.tree_check_thresholds(thr, ord_, w))

    np.savez_compressed(os.path.join(HERE, "forest.npz"), **out)
    print("wrote forest.npz with", len(out), "arrays")
    families(ref)
    init_vectors(ref)
    double_vectors(ref)


LINEAR_CASES = [
    # kind, B, C, inner, T, depth, extra, O, Cv (0 = no vector: plain fused linear)
    ("tree", 7, 9, (), 5, 3, (), 4, 0),
    ("fern", 5, 11, (3,), 4, 4, (2,), 3, 0),
    ("tree", 6, 5, (2,), 4, 3, (2,), 3, 4),
    ("fern", 6, 5, (), 4, 3, (), 2, 3),
]

CONV_CASES = [
    # dims, x shape, Co, depth, extra, kernel, stride, padding, dilation
    (1, (2, 3, 9), 4, 2, (), (3,), (1,), (1,), (1,)),
    (2, (2, 3, 6, 7), 4, 3, (), (3, 3), (1, 1), (1, 1), (1, 1)),
    (2, (1, 2, 8, 9), 3, 2, (2,), (2, 3), (2, 1), (1, 2), (2, 1)),
    (3, (1, 2, 5, 6, 4), 2, 2, (), (2, 3, 2), (1, 2, 1), (1, 0, 1), (1, 1, 2)),
]

PATCH_CASES = [((2, 3, 7, 9), (2, 3), (1, 0)), ((1, 2, 8, 8), (4, 4), (2, 2)), ((1, 2, 5, 6, 7), (2, 3, 2), (1, 1, 0))]


def double_vectors(ref):
    """The forest cases once more in double precision -> forest64.npz (forward, maps, backward)."""
    out = {}
    for idx, (seed, kind, B, C, inner, T, depth, extra, adv) in enumerate(forest_cases()):
        gen = torch.Generator().manual_seed(9000 + seed)
        N = decisions(kind, depth)
        x = torch.randn((B, C) + tuple(inner), generator=gen, dtype=torch.float64)
        thr = torch.rand((T, N), generator=gen, dtype=torch.float64) * 6 - 3
        ord_ = torch.randint(0, C, (T, N), generator=gen)
        w = torch.randn((T, 2 ** depth) + tuple(extra), generator=gen, dtype=torch.float64)
        if adv:
            x = torch.round(x * 2) / 2
            thr = torch.round(thr * 2) / 2
            ord_[:, : min(N, 3)] = ord_[:, :1]
        f = getattr(ref, kind + "_forward")(x, thr, ord_, w)
        g = torch.randn(f.shape, generator=gen, dtype=torch.float64)
        gx, gthr, _, gw = getattr(ref, kind + "_backward")(x, True, thr, True, ord_, False, w, True, g)
        leaf = getattr(ref, kind + "_leafmap")(x, thr, ord_, w)
        margin, mord = getattr(ref, kind + "_marginmap")(x, thr, ord_, w)
        reach = getattr(ref, kind + "_reachability")(x, thr, ord_, w)
        p = "forest%02d_" % idx
        out[p + "kind"] = np.array(kind)
        for name, t in [("x", x), ("thr", thr), ("ord", ord_), ("w", w), ("g", g), ("out", f), ("gx", gx),
                        ("gthr", gthr), ("gw", gw), ("margin", margin), ("margin_ord", mord)]:
            out[p + name] = t.numpy()
        out[p + "leaf"] = leaf.numpy().astype(np.int64)
        out[p + "reach"] = reach.numpy().astype(np.int64)
    out["forest_count"] = np.array(len(forest_cases()))
    np.savez_compressed(os.path.join(HERE, "forest64.npz"), **out)
    print("wrote forest64.npz with", len(out), "arrays")


def families(ref, dtype=torch.float32, filename="families.npz"):
    """Fused linear, image+vector fusion, convolution, contract/expand and trie vectors -> families.npz; with
    dtype=torch.float64 the same cases (the same values, widened) in double precision -> families64.npz."""
    out = {}
    for idx, (kind, B, C, inner, T, depth, extra, O, Cv) in enumerate(LINEAR_CASES):
        gen = torch.Generator().manual_seed(500 + idx)
        N = decisions(kind, depth)
        x = torch.randn((B, C) + inner, generator=gen).to(dtype)
        thr = (torch.rand((T, N), generator=gen) * 6 - 3).to(dtype)
        ord_ = torch.randint(0, C + Cv, (T, N), generator=gen)
        w = torch.randn((T, 2 ** depth) + extra, generator=gen).to(dtype)
        lin = torch.randn((O, T), generator=gen).to(dtype)
        bias = torch.randn(O, generator=gen).to(dtype)
        p = "linear%02d_" % idx
        out[p + "kind"] = np.array(kind)
        tensors = [("x", x), ("thr", thr), ("ord", ord_), ("w", w), ("lin", lin), ("bias", bias)]
        if Cv:
            vec = torch.randn((B, Cv), generator=gen).to(dtype)
            tensors.append(("vec", vec))
            f = getattr(ref, kind + "_fusion_fused_linear_forward")(x, vec, thr, ord_, w, lin, bias)
            g = torch.randn(f.shape, generator=gen).to(dtype)
            grads = getattr(ref, kind + "_fusion_fused_linear_backward")(x, True, vec, True, thr, True, ord_, False, w,
                                                                         True, lin, True, bias, True, g)
            names = ["gx", "gvec", "gthr", None, "gw", "glin", "gbias"]
            ff = getattr(ref, kind + "_fusion_forward")(x, vec, thr, ord_, w)
            g2 = torch.randn(ff.shape, generator=gen).to(dtype)
            fg = getattr(ref, kind + "_fusion_backward")(x, True, vec, True, thr, True, ord_, False, w, True, g2)
            tensors += [("fusion_out", ff), ("fusion_g", g2), ("fusion_gx", fg[0]), ("fusion_gvec", fg[1]),
                        ("fusion_gthr", fg[2]), ("fusion_gw", fg[4])]
        else:
            f = getattr(ref, kind + "_fused_linear_forward")(x, thr, ord_, w, lin, bias)
            g = torch.randn(f.shape, generator=gen).to(dtype)
            grads = getattr(ref, kind + "_fused_linear_backward")(x, True, thr, True, ord_, False, w, True, lin, True,
                                                                  bias, True, g)
            names = ["gx", "gthr", None, "gw", "glin", "gbias"]
        tensors += [("out", f), ("g", g)] + [(n, t) for n, t in zip(names, grads) if n is not None]
        for name, t in tensors:
            out[p + name] = t.numpy()
    out["linear_count"] = np.array(len(LINEAR_CASES))

    for kidx, kind in enumerate(("tree", "fern")):
        for cidx, (dims, xs, Co, depth, extra, kernel, stride, padding, dilation) in enumerate(CONV_CASES):
            gen = torch.Generator().manual_seed(700 + 10 * kidx + cidx)
            Ci, N, cells = xs[1], decisions(kind, depth), int(np.prod(kernel))
            x = torch.randn(xs, generator=gen).to(dtype)
            thr = (torch.rand((Co, Ci, N), generator=gen) * 2 - 1).to(dtype)
            ord_ = torch.randint(0, cells, (Co, Ci, N), generator=gen)
            w = torch.randn((Co, Ci, 2 ** depth) + extra, generator=gen).to(dtype)
            geometry = [list(kernel), list(stride), list(padding), list(dilation)]
            f = getattr(ref, "%s_conv%dd_forward" % (kind, dims))(x, thr, ord_, w, *geometry)
            g = torch.randn(f.shape, generator=gen).to(dtype)
            gx, gthr, _, gw = getattr(ref, "%s_conv%dd_backward" % (kind, dims))(x, True, thr, True, ord_, False, w, True,
                                                                               g, *geometry)
            p = "conv%02d_" % (len(CONV_CASES) * kidx + cidx)
            out[p + "kind"] = np.array(kind)
            out[p + "geometry"] = np.array(geometry)
            for name, t in [("x", x), ("thr", thr), ("ord", ord_), ("w", w), ("out", f), ("g", g), ("gx", gx),
                            ("gthr", gthr), ("gw", gw)]:
                out[p + name] = t.numpy()
    out["conv_count"] = np.array(2 * len(CONV_CASES))

    for idx, (xs, window, padding) in enumerate(PATCH_CASES):
        x = torch.randint(-100, 100, xs, generator=torch.Generator().manual_seed(900 + idx)).to(torch.int16)
        c = ref.contract(x, list(window), list(padding))
        p = "patch%02d_" % idx
        out[p + "x"], out[p + "window"], out[p + "padding"] = x.numpy(), np.array(window), np.array(padding)
        out[p + "contracted"], out[p + "expanded"] = c.numpy(), ref.expand(c, list(padding)).numpy()
    out["patch_count"] = np.array(len(PATCH_CASES))

    # hinge tries (CPU only in the reference): weights sit on the internal vertices
    for idx, (B, C, inner, T, depth, extra) in enumerate([(9, 7, (), 5, 3, ()), (4, 6, (3,), 3, 4, (2,))]):
        gen = torch.Generator().manual_seed(950 + idx)
        N = 2 ** depth - 1
        x = torch.randn((B, C) + inner, generator=gen).to(dtype)
        thr = (torch.rand((T, N), generator=gen) * 4 - 2).to(dtype)
        ord_ = torch.randint(0, C, (T, N), generator=gen)
        w = torch.randn((T, N) + extra, generator=gen).to(dtype)
        f = ref.trie_forward(x, thr, ord_, w)
        g = torch.randn(f.shape, generator=gen).to(dtype)
        gx, gthr, _, gw = ref.trie_backward(x, True, thr, True, ord_, False, w, True, g)
        p = "trie%02d_" % idx
        for name, t in [("x", x), ("thr", thr), ("ord", ord_), ("w", w), ("out", f), ("g", g), ("gx", gx),
                        ("gthr", gthr), ("gw", gw)]:
            out[p + name] = t.numpy()
    out["trie_count"] = np.array(2)
    np.savez_compressed(os.path.join(HERE, filename), **out)
    print("wrote", filename, "with", len(out), "arrays")


INIT_CASES = [
    # family, B, C, inner, T, depth, quantised (ties), dtype
    ("tree", 37, 5, (), 4, 3, False, torch.float32),
    ("tree", 6, 4, (3,), 3, 4, False, torch.float32),   # fewer samples than vertices: some are never reached
    ("tree", 40, 3, (), 3, 3, True, torch.float32),     # many equal values
    ("tree", 1, 3, (), 2, 2, False, torch.float32),
    ("tree", 2, 3, (), 2, 2, False, torch.float32),
    ("tree", 19, 4, (2,), 2, 3, False, torch.float64),
    ("fern", 21, 6, (), 5, 4, False, torch.float32),
    ("fern", 8, 3, (2, 2), 3, 3, True, torch.float32),
    ("trie", 25, 5, (), 3, 3, False, torch.float32),
    ("trie", 12, 4, (2,), 2, 2, True, torch.float32),
]


def init_vectors(ref):
    """Median initialisation of thresholds (tree, fern, trie) -> init.npz."""
    out = {}
    for idx, (family, B, C, inner, T, depth, quantised, dtype) in enumerate(INIT_CASES):
        gen = torch.Generator().manual_seed(700 + idx)
        N = depth if family == "fern" else 2 ** depth - 1
        x = torch.randn((B, C) + inner, generator=gen).to(dtype)
        if quantised:
            x = torch.round(x * 2) / 2
        thr = (torch.rand((T, N), generator=gen) * 6 - 3).to(dtype)
        ord_ = torch.randint(0, C, (T, N), generator=gen)
        w = torch.zeros((T, N if family == "trie" else 2 ** depth), dtype=dtype)
        after = thr.clone()
        ok = getattr(ref, family + "_init_medians")(x, after, ord_, w)
        p = "init%02d_" % idx
        out[p + "family"] = np.array(family)
        for name, t in [("x", x), ("thr", thr), ("ord", ord_), ("w", w), ("after", after)]:
            out[p + name] = t.numpy()
        out[p + "ok"] = np.array(bool(ok))
    out["count"] = np.array(len(INIT_CASES))
    np.savez_compressed(os.path.join(HERE, "init.npz"), **out)
    print("wrote init.npz with", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "double":  # only the double precision files
        double_vectors(build_ref.load())
        families(build_ref.load(), torch.float64, "families64.npz")
    else:
        main()
