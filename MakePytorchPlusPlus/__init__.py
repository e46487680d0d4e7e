"""Drop-in for the reference's package name (``setup.py:12-13``, ``__init__.py:1-7``): the same
eight names, served by ``pytorch_winoconv_b200``.  Importing it also registers the compiled
module under its reference name ``MakePytorchBackend``."""
from pytorch_winoconv_b200._backend import load as _load

_backend = _load()
AddGPU, Foo, WinoSplit, WinoConcat, DWM = (_backend.AddGPU, _backend.Foo, _backend.WinoSplit,
                                           _backend.WinoConcat, _backend.DWM)

from pytorch_winoconv_b200.Add import add_gpu  # noqa: E402
from pytorch_winoconv_b200.Split_and_Concat import wino_concat, wino_split  # noqa: E402

__all__ = ["AddGPU", "Foo", "WinoSplit", "WinoConcat", "DWM", "add_gpu", "wino_split", "wino_concat"]
