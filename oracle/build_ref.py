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

Usage:  python oracle/build_ref.py [--reference /path/to/HingeTreeForTorch] [--jobs N] [--gpu]

With ``--gpu`` the reference is built a second time with its CUDA kernels (``build_gpu``), as the second
baseline bench.py times when the file is present.

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


# The reference's GPU translation units (the torch.cuda.is_available() branch of its setup.py:29-37).
GPU_MODULE = "hingetree_ref_gpu"
GPU_SOURCES = [
    "hingetree_gpu.cu", "hingetree_sparse_gpu.cu", "ImageToMatrix_gpu.cu", "hingetree_conv_gpu.cu",
    "hingetree_fused_linear_gpu.cu", "hingetree_fusion_gpu.cu", "expand_gpu.cu",
]


def gpu_so_path():
    return os.path.join(OUT, GPU_MODULE + sysconfig.get_config_var("EXT_SUFFIX"))


def build_gpu(reference, jobs=8, force=False):
    """The unmodified reference WITH its CUDA kernels (``-DWITH_CUDA=1``, as its setup.py does when a GPU is
    present), compiled for sm_100 into ``oracle/_ref/hingetree_ref_gpu*.so``: the reference's own GPU code as
    a second baseline beside its CPU code.  nvcc cross-compiles, so this runs on a machine without a GPU.
    Callers keep the batch at or below 524 280 rows: the reference launches ``gridDim.y = B / 8`` unchecked
    (hingetree_gpu.cu:491-495)."""
    from torch.utils import cpp_extension as ce
    import torch

    target = gpu_so_path()
    cpu_srcs = [os.path.join(reference, s) for s in SOURCES]
    gpu_srcs = [os.path.join(reference, s) for s in GPU_SOURCES]
    if not all(os.path.exists(s) for s in cpu_srcs + gpu_srcs):
        raise FileNotFoundError("reference sources not found under %s" % reference)
    if os.path.exists(target) and not force:
        if os.path.getmtime(target) >= max(os.path.getmtime(s) for s in cpu_srcs + gpu_srcs):
            return target
    gpu_out = os.path.join(OUT, "gpu")
    os.makedirs(gpu_out, exist_ok=True)
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    cxx = os.environ.get("CXX", "g++")
    try:
        paths = ce.include_paths(device_type="cuda")
    except TypeError:  # older signature
        paths = ce.include_paths(True)
    inc = []
    for p in paths + [os.path.join(cuda_home, "include"), sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    defines = ["-DWITH_CUDA=1", "-DTORCH_EXTENSION_NAME=" + GPU_MODULE, "-DTORCH_API_INCLUDE_EXTENSION_H",
               "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi]

    def compile_one(src):
        obj = os.path.join(gpu_out, os.path.basename(src) + ".o")
        if src.endswith(".cu"):
            cmd = [nvcc, "-O2", "-std=c++17", "-w", "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr",
                   "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
                   "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-Xcompiler", "-fPIC"] + defines + inc
        else:
            cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-w"] + defines + inc
        subprocess.run(cmd + ["-c", src, "-o", obj], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(compile_one, gpu_srcs + cpu_srcs))
    link = [cxx, "-shared", "-o", target] + objs
    for cand in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/usr/lib64/libstdc++.so.6"):
        if os.path.exists(cand):
            link.append(cand)
            break
    for d in ce.library_paths(device_type="cuda") + [os.path.join(cuda_home, "lib64")]:
        link += ["-L" + d, "-Wl,-rpath," + d]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
    subprocess.run(link, check=True)
    return target


def load_gpu():
    """Import the reference built with its GPU kernels (raises ImportError if it was never built)."""
    import importlib.util
    import torch  # noqa: F401
    path = gpu_so_path()
    if not os.path.exists(path):
        raise ImportError("reference GPU build not present: run python oracle/build_ref.py --gpu")
    spec = importlib.util.spec_from_file_location(GPU_MODULE, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


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
    ap.add_argument("--gpu", action="store_true", help="also build the reference with its CUDA kernels (several minutes)")
    a = ap.parse_args()
    print(build(a.reference, a.jobs, a.force))
    print(extract_trained_forests(a.reference))
    if a.gpu:
        print(build_gpu(a.reference, a.jobs, a.force))
    sys.exit(0)
