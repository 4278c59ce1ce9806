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


if __name__ == "__main__":
    main()
