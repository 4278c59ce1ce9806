"""Build recipe for the unmodified reference CPU implementation (test infrastructure only).

Compiles the reference's own C++ translation units, in place from the read-only reference
checkout, into ``oracle/_ref/hingetree_ref_cpp*.so``.  Nothing from the reference is copied
into this repository: only object files and the shared library are written, and only under
``oracle/_ref/`` (git-ignored).

The module name is chosen by the ``TORCH_EXTENSION_NAME`` macro (the reference's
``PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)`` in hingetree.cpp:1962), so the result can be
imported next to this repository's own ``hingetree_cpp``.  The build is CPU only (the
reference's ``WITH_CUDA`` macro stays undefined, as in the ``CppExtension`` branch of its
setup.py:47-56) and uses the same ``-O2`` the reference's setup.py:24 passes.

Usage:  python oracle/build_ref.py [--reference /path/to/HingeTreeForTorch] [--jobs N]

The product never imports this module or its output; only tests, the smoke check and the
CPU-baseline legs of bench.py do, as the checker.
"""
import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULE = "hingetree_ref_cpp"

# Translation units of the reference's CPU build (its setup.py:22).
SOURCES = [
    "hingetree.cpp", "hingetree_sparse.cpp", "hingetrie.cpp", "ImageToMatrix.cpp",
    "hingetree_conv.cpp", "hingetree_fused_linear.cpp", "hingetree_fusion.cpp",
    "expand.cpp", "Timer.cpp",
]


def so_path():
    return os.path.join(OUT, MODULE + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference, jobs=8, force=False):
    from torch.utils import cpp_extension as ce
    import torch

    target = so_path()
    srcs = [os.path.join(reference, s) for s in SOURCES]
    if not all(os.path.exists(s) for s in srcs):
        raise FileNotFoundError("reference sources not found under %s" % reference)
    if os.path.exists(target) and not force:
        newest = max(os.path.getmtime(s) for s in srcs)
        if os.path.getmtime(target) >= newest:
            return target
    os.makedirs(OUT, exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = [cxx, "-O2", "-std=c++17", "-fPIC", "-w",
              "-DTORCH_EXTENSION_NAME=" + MODULE, "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi] + inc

    def compile_one(src):
        obj = os.path.join(OUT, os.path.basename(src) + ".o")
        subprocess.run(common + ["-c", src, "-o", obj], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(compile_one, srcs))
    libdirs = ce.library_paths()
    link = [cxx, "-shared", "-o", target] + objs
    # name the shared C++ runtime first, so that a static libstdc++.a is never pulled in
    for cand in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/usr/lib64/libstdc++.so.6"):
        if os.path.exists(cand):
            link.append(cand)
            break
    for d in libdirs:
        link += ["-L" + d, "-Wl,-rpath," + d]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    subprocess.run(link, check=True)
    return target


def trained_forest_path():
    return os.path.join(OUT, "trained_forests.npz")


def extract_trained_forests(reference, limit=2):
    """Read the hinge forest parameters (thresholds, ordinals, leaf weights) out of the trained
    checkpoints the reference ships for its renal-cell-carcinoma example (rcc/Models/*/epoch_*.pt:
    100 trees of depth 7 over 100 channels, 8 x 8 outputs per leaf, rcc/Net.py:64) into
    ``oracle/_ref/trained_forests.npz`` so that the parity tests can use realistic, trained
    parameters wherever ``oracle/_ref`` travels.  Like everything under ``oracle/_ref`` the file is
    git-ignored: nothing of the reference enters the history."""
    import glob

    import numpy as np
    import torch

    files = sorted(glob.glob(os.path.join(reference, "rcc", "Models", "*", "epoch_*.pt")))[:limit]
    if not files:
        return None
    target = trained_forest_path()
    if os.path.exists(target) and os.path.getmtime(target) >= max(os.path.getmtime(f) for f in files):
        return target
    os.makedirs(OUT, exist_ok=True)
    arrays = {"count": np.int64(len(files))}
    for n, f in enumerate(files):
        state = torch.load(f, map_location="cpu", weights_only=True)
        arrays["thr%d" % n] = state["forest.thresholds"].float().numpy()
        arrays["ord%d" % n] = state["forest.ordinals"].long().numpy()  # old checkpoints store them as float32
        arrays["w%d" % n] = state["forest.weights"].float().numpy()
    np.savez(target, **arrays)
    return target


def load():
    """Import the built reference module (raises ImportError if it was never built)."""
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    path = so_path()
    if not os.path.exists(path):
        raise ImportError("reference oracle not built: run python oracle/build_ref.py")
    spec = importlib.util.spec_from_file_location(MODULE, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("HINGETREE_REFERENCE"), required="HINGETREE_REFERENCE" not in os.environ,
                    help="checkout of NIH-MIP/HingeTreeForTorch (or set HINGETREE_REFERENCE)")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.jobs, a.force))
    print(extract_trained_forests(a.reference))
    sys.exit(0)
