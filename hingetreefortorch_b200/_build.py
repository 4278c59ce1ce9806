"""In-tree build of the native parts: the C-ABI CUDA library and the torch extension.

  libhingetree_b200.so   nvcc, sm_100a only: every kernel and the extern "C" entry points
  hingetree_cpp.*.so     g++: the torch/pybind host layer, linked against the library

Both land next to this file so that they are found (and seen to be loaded) from the source
tree.  nvcc cross-compiles without a GPU, so this also runs on a CPU-only build machine.
"""
import glob
import os
import subprocess
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ = os.path.join(PKG, "build")

LIB_NAME = "libhingetree_b200.so"
EXT_NAME = "hingetree_cpp"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def library_path():
    return os.path.join(PKG, LIB_NAME)


def extension_path():
    return os.path.join(PKG, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _nvcc():
    home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _shared_libstdcxx():
    """Full path of the shared libstdc++, put on link lines explicitly.

    Some toolchain layouts carry a dangling libstdc++.so next to libstdc++.a, and the linker
    then silently links the static archive into the shared object (two C++ runtimes in one
    process: iostreams crash).  Naming the shared library first leaves the archive nothing to add.
    """
    try:
        out = subprocess.run(["ldconfig", "-p"], capture_output=True, text=True).stdout
        for line in out.splitlines():
            if "libstdc++.so.6" in line and "x86-64" in line and "=>" in line:
                return [line.split("=>")[1].strip()]
    except OSError:
        pass
    for cand in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/usr/lib64/libstdc++.so.6"):
        if os.path.exists(cand):
            return [cand]
    return []


def build_library(force=False, verbose=False):
    """Compile csrc/*.cu for sm_100a and link libhingetree_b200.so."""
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    target = library_path()
    os.makedirs(OBJ, exist_ok=True)
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        if force or _newer(obj, [src] + headers):
            subprocess.run([_nvcc()] + flags + ["-I" + INCLUDE, "-I" + CSRC, "-c", src, "-o", obj], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _newer(target, objs):
        subprocess.run([_nvcc(), "-Wno-deprecated-gpu-targets", "-shared", "-o", target] + objs + ["-lcudart"], check=True)
    return target


def build_extension(force=False):
    """Compile the pybind/torch host layer and link it against the C-ABI library."""
    import torch
    from torch.utils import cpp_extension as ce

    sources = sorted(glob.glob(os.path.join(CSRC, "hingetree_cpp*.cpp")))
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(INCLUDE, "*.h"))
    target = extension_path()
    os.makedirs(OBJ, exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    inc = ["-I" + INCLUDE, "-I" + CSRC]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]:
        inc += ["-isystem", p]
    common = [cxx, "-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function",
              "-DTORCH_EXTENSION_NAME=" + EXT_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + inc

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        if force or _newer(obj, [src] + headers):
            subprocess.run(common + ["-c", src, "-o", obj], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _newer(target, objs + [library_path()]):
        link = [cxx, "-shared", "-o", target] + objs + _shared_libstdcxx() + ["-L" + PKG, "-lhingetree_b200", "-Wl,-rpath,$ORIGIN"]
        for d in ce.library_paths() + [os.path.join(cuda_home, "lib64")]:
            link += ["-L" + d, "-Wl,-rpath," + d]
        link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        subprocess.run(link, check=True)
    return target


def build_all(force=False):
    return build_library(force), build_extension(force)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared memory usage")
    ap.add_argument("--library-only", action="store_true")
    a = ap.parse_args()
    print(build_library(a.force, a.verbose))
    if not a.library_only:
        print(build_extension(a.force))
