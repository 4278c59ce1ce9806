"""hingetreefortorch_b200: sm_100a evaluation path of random hinge forests and ferns.

Layers, bottom up:
  libhingetree_b200.so   hand-written CUDA kernels behind the C ABI of include/hingetree_b200.h
  hingetree_cpp          torch extension with the reference's operator names and checks
  HingeTree              torch.autograd.Function layer (same class names as the reference)
  RandomHingeForest      nn.Module layer (same class names and constructor arguments)

Importing this package does not load native code; `hingetreefortorch_b200.HingeTree` and
`hingetreefortorch_b200.RandomHingeForest` do, and fail loudly when it was not built.
"""
__version__ = "0.1.0"

__all__ = ["build", "install_dropin"]


def build(force=False):
    """Compile the CUDA library and the torch extension in-tree."""
    from . import _build
    return _build.build_all(force)


def install_dropin():
    from ._ext import install_dropin as _install
    _install()


def __getattr__(name):
    if name in ("HingeTree", "RandomHingeForest", "distributed"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)
