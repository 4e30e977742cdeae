"""B200-native programmable collectives and communication/computation overlap.

Sub-packages load on first use (``pccl_b200.lang``, ``.engine``, ``.synth``, ``.ops``, ``.nn``, ``.models``,
``.parallel``, ``.utils``), so importing the package costs nothing and works on a box without a GPU.
"""
import importlib

__version__ = "0.1.0"
_SUBMODULES = ("lang", "engine", "synth", "ops", "nn", "models", "parallel", "utils")


def __getattr__(name):
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_SUBMODULES))
