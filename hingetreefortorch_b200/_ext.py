"""Loads the in-tree torch extension `hingetree_cpp` (the drop-in for the reference's module).

There is no pure-Python or CPU fallback: when the extension or the CUDA library was not
built, importing this module raises.
"""
import ctypes
import importlib.util
import os
import sys

import torch  # noqa: F401  (libtorch must be resident before the extension is opened)

from . import _build


def _load():
    lib, ext = _build.library_path(), _build.extension_path()
    for path in (lib, ext):
        if not os.path.exists(path):
            raise ImportError("%s is missing: build it with `python -m hingetreefortorch_b200._build` "
                              "(there is no fallback path)" % path)
    ctypes.CDLL(lib, mode=ctypes.RTLD_GLOBAL)
    spec = importlib.util.spec_from_file_location(_build.EXT_NAME, ext)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


hingetree_cpp = _load()


def install_dropin():
    """Make `import hingetree_cpp`, `import HingeTree` and `import RandomHingeForest` resolve to this package."""
    from . import HingeTree, RandomHingeForest
    sys.modules["hingetree_cpp"] = hingetree_cpp
    sys.modules["HingeTree"] = HingeTree
    sys.modules["RandomHingeForest"] = RandomHingeForest
