"""Loader of the compiled operator module ``MakePytorchBackend`` (reference: ``setup.py:16``,
``pybind/bind.cpp:11``).  Fails loudly when it has not been built: there is no Python fallback."""
import importlib
import os
import sys

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))


def load():
    name = __package__ + ".MakePytorchBackend"
    if name in sys.modules:
        return sys.modules[name]
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    try:
        mod = importlib.import_module(name)
    except ImportError as e:
        raise ImportError(
            "pytorch_winoconv_b200.MakePytorchBackend is not built (or libwinoconv_b200.so is missing). "
            "Run `python -m pytorch_winoconv_b200.build`; there is no fallback implementation. "
            f"Original error: {e}") from e
    sys.modules.setdefault("MakePytorchBackend", mod)
    return mod
